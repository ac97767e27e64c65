#!/usr/bin/env python
"""Headline benchmark: Qwen3-8B `jetlong_fused` full-model prefill throughput (tok/s) at 131072
tokens on B200, plus the decode-attention microbench at 131072 keys, with the roofline of the
dominant kernel and the reference's CPU path timed beside it.

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference            # the reference's eager composition on the host cores

One "step" is one prefill forward `model(input_ids, use_cache=True)` over a fresh 131072-token
prompt (the reference's own protocol: scripts/throughput/bench_prefill_throughput.py:83-95 in the
Jet-Long repository), random-init bf16 weights, uniform random token ids.  With N > 1 the prompt is
sequence-parallel: tokens (projections, MLP, logits) and the KV cache are sharded block-cyclically
over the ranks; per layer the base-rotated queries are all-gathered, every rank attends all query
stripes to its own key stripe, and the partial (O, LSE) pairs go back to the ranks that own the
rows (all-to-all) where the merge kernel combines them (strong scaling: the prompt stays 131072 tokens).
Rank 0 prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path[:0] = [os.path.join(ROOT, "jet-long_b200")]

import torch  # noqa: E402

MODEL_DIMS = {
    "qwen3-8b": dict(variant="Qwen3-8B-Base-jetlong_fused"),
    "qwen3-4b": dict(variant="Qwen3-4B-Base-jetlong_fused"),
    "qwen3-1.7b": dict(variant="Qwen3-1.7B-Base-jetlong_fused"),
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"], bf16_tflops_sustained=p["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


def model_config(name: str, w: int, w_0: int, layers: int | None):
    from transformers.models.qwen3.configuration_qwen3 import Qwen3Config
    with open(os.path.join(ROOT, "jet-long_b200", "model_configs", MODEL_DIMS[name]["variant"], "config.json")) as f:
        d = json.load(f)
    d.pop("auto_map", None)
    d.pop("architectures", None)
    d["jetlong"] = dict(d["jetlong"], w=w, w_0=w_0)
    if layers:
        d["num_hidden_layers"] = layers
        d["max_window_layers"] = layers
    cfg = Qwen3Config(**d)
    cfg._attn_implementation = "sdpa"
    return cfg


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.idx)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True).start()
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        busy = sorted(sm)[len(sm) // 2:] if sm else []
        return dict(sm_mhz=statistics.median(busy) if busy else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


# --------------------------------------------------------------------------------------------------
# CPU baseline: the oracle (a restatement of the reference's eager composition) on the host cores
# --------------------------------------------------------------------------------------------------

def cpu_prefill_sample(S: int, dims: dict, w_0: int, G: int, blocks: int = 24):
    """Time a bounded sample of the prefill workload on the CPU (about 10-20 s at the default size) and
    extrapolate to tokens/s.

    Attention: the oracle's two-branch bifocal composition for `blocks` 128-row query blocks spread evenly over
    the prompt (the last one ends at row S) of 8 query heads (one per kv head) over their full causal key
    range, scaled by (query heads / 8) x (all causal pairs / sampled pairs).  The RoPE / regroup of the
    operands is timed apart and scaled by rows, because the workload rotates every row once per layer, not once
    per query block.  Dense layers: the fp32 projections + MLP of one layer on 1024 tokens and a slice of the
    lm_head on 256 tokens, scaled to S tokens and all layers."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import jetlong_oracle as orc
    H, Hk, D, L = dims["heads"], dims["kv_heads"], 128, dims["layers"]
    hidden, inter, vocab = dims["hidden"], dims["inter"], dims["vocab"]
    torch.manual_seed(0)
    inv = orc.default_inv_freq()
    blocks = max(1, min(blocks, S // 128))
    k_all = torch.randn(1, S, Hk, D)
    v_all = torch.randn(1, S, Hk, D)
    t_attn, t_rot, pairs, rot_rows = 0.0, 0.0, 0, 0
    starts = [(i + 1) * S // blocks - 128 for i in range(blocks)]
    for q0 in starts:
        n_k = q0 + 128
        k, v = k_all[:, :n_k], v_all[:, :n_k]
        q = torch.randn(1, 128, Hk, D)
        qp = (torch.arange(128) + q0).view(1, -1)
        kp = torch.arange(n_k).view(1, -1)
        t0 = time.perf_counter()
        qb, qg, kb, kg = orc.jetlong_operands(q, k, q_positions=qp, k_positions=kp, group_size=G, inv_freq=inv)
        t1 = time.perf_counter()
        orc.jetlong_prefill(qb, qg, kb, kg, v, seqstart=q0, w0=w_0)
        t2 = time.perf_counter()
        t_rot += t1 - t0
        t_attn += t2 - t1
        pairs += 128 * q0 + 128 * 129 // 2
        rot_rows += (n_k + 128) * Hk
    total_pairs = S * (S + 1) // 2
    attn_layer = t_attn * (H / Hk) * (total_pairs / pairs) + t_rot * (S * (H + Hk) / rot_rows)
    n_tok = 1024
    x = torch.randn(n_tok, hidden)
    ws = [torch.randn(hidden, H * D), torch.randn(hidden, 2 * Hk * D), torch.randn(H * D, hidden),
          torch.randn(hidden, 2 * inter), torch.randn(inter, hidden)]
    t0 = time.perf_counter()
    a = x @ ws[0]; _ = x @ ws[1]; _ = a @ ws[2]
    u = x @ ws[3]
    _ = (torch.nn.functional.silu(u[:, :inter]) * u[:, inter:]) @ ws[4]
    t_dense = time.perf_counter() - t0
    dense_layer = t_dense * (S / n_tok)
    xh = torch.randn(256, hidden)
    vslice = min(vocab, 16384)
    wv = torch.randn(hidden, vslice)
    t0 = time.perf_counter()
    _ = xh @ wv
    t_head = time.perf_counter() - t0
    head = t_head * (S / 256) * (vocab / vslice)
    total = L * (attn_layer + dense_layer) + head
    return dict(tok_s=S / total, est_total_s=total, attn_s=L * attn_layer, dense_s=L * dense_layer + head,
                sample_s=t_attn + t_rot + t_dense + t_head, cores=torch.get_num_threads(),
                sample=(f"oracle bifocal attention for {blocks} query blocks of 128 rows (ending at rows "
                        f"{starts[0] + 128}, ..., {starts[-1] + 128}) x {Hk} heads over their causal key range, operand RoPE/regroup "
                        f"timed apart; one layer's fp32 projections/MLP on {n_tok} tokens; a {vslice}-column slice of the lm_head on "
                        f"256 tokens; extrapolated by causal-pair count, head count, rows, tokens and {L} layers"))


def model_dims(cfg):
    return dict(heads=cfg.num_attention_heads, kv_heads=cfg.num_key_value_heads, layers=cfg.num_hidden_layers,
                hidden=cfg.hidden_size, inter=cfg.intermediate_size, vocab=cfg.vocab_size)


def run_reference(args):
    """The reference's CPU path for the same config on all host cores: rank 0 alone works (the other ranks of a
    torchrun launch exit at once).  The sample is deterministic, so a few repeats are enough: one small warm-up
    and best of min(steps, 3) full samples, whatever --steps / --warmup say (they are echoed in the line)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # torch.distributed.run exports OMP_NUM_THREADS=1 to its workers; the CPU baseline is meant to use the box
    torch.set_num_threads(os.cpu_count() or 1)
    cfg = model_config(args.model, args.w, args.w0, args.layers)
    G = max(1, math.ceil(args.seq / args.w))
    if args.warmup > 0:
        cpu_prefill_sample(min(args.seq, 8192), model_dims(cfg), min(args.w0, 2048), G, blocks=8)
    res = [cpu_prefill_sample(args.seq, model_dims(cfg), args.w0, G) for _ in range(max(1, min(args.steps, 3)))]
    best = max(res, key=lambda r: r["tok_s"])
    value = float(f"{best['tok_s']:.3g}")
    line = dict(metric="prefill_tok_per_s", value=value, unit="tok/s", n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=best["est_total_s"] * 1e3, higher_is_better=True, scaling="strong",
                vs_baseline=None, dtype="f32", data="synthetic", impl="reference",
                config=workload_config(args, cfg, G),
                cpu_baseline=dict(value=value, unit="tok/s", cores=best["cores"], kind="port", sample=best["sample"],
                                  samples_timed=len(res), spread=[float(f"{r['tok_s']:.3g}") for r in res]),
                e2e=dict(value=value, unit="tok/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                note="reference fused kernels are gated to sm_90 and need flash_attn.cute (not installed): the reference's "
                     "eager composition (restated in oracle/) is timed on the host cores on a bounded sample and extrapolated; "
                     "run-to-run spread of the sample is 5-20 %, so the value carries two to three significant digits")
    print(json.dumps(line), flush=True)


def workload_config(args, cfg, G, sp_mode="kv_gather"):
    return dict(workload=f"{args.model} jetlong_fused full-model prefill, batch 1, {args.seq} tokens",
                layers=cfg.num_hidden_layers, heads=cfg.num_attention_heads, kv_heads=cfg.num_key_value_heads,
                head_dim=128, hidden=cfg.hidden_size, w=args.w, w_0=args.w0, group_size=G,
                logits="all positions (reference bench protocol)" if args.logits_to_keep == 0 else f"last {args.logits_to_keep}",
                l2="inputs and weights far exceed the 126 MB L2; decode microbench flushes L2 (256 MB write + 256 MB read) between iterations",
                parallelism=(f"sequence-parallel x{args.gpus}: tokens and KV cache block-cyclic over ranks (block {SP_BLOCK}); "
                             "per layer all-gather of K_base and V, local regroup, one launch of this rank's query stripe "
                             "against all keys" if sp_mode == "kv_gather" else
                             f"sequence-parallel x{args.gpus}: tokens and KV cache block-cyclic over ranks (block {SP_BLOCK}), "
                             "Q all-gather, partial (O,LSE) all-to-all + N-way merge") if args.gpus > 1 else "single GPU")


# --------------------------------------------------------------------------------------------------
# decode-attention microbench (the reference's protocol: CUDA graph, 256 MB L2 flush, median)
# --------------------------------------------------------------------------------------------------

def decode_microbench(peaks, shard, iters=20, ctx=131072, w0=32768, batches=(1, 8), variants_wanted=None):
    from jetlm.kernels import cute_jetlong_backend as backend, jetlong_ops as ops
    out = {}
    H, Hk, D, G = 32, 8, 128, 4
    world = shard.world if shard is not None else 1
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    flush_rd = torch.zeros(256 << 20, dtype=torch.uint8, device="cuda")

    def cold_l2():
        # evict everything (256 MB write), then read another 256 MB so the evicted dirty lines are written back
        # before the timed kernel starts instead of competing with its loads: L2 is cold AND clean
        flush.zero_()
        flush_rd.max()

    inv = 1.0 / (1.0e6 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    exchange_used = {}
    for B in batches:
        torch.manual_seed(0)
        q = torch.randn(B, 1, H, D, device="cuda").bfloat16()
        qg = torch.randn(B, 1, H, D, device="cuda").bfloat16()
        kc = torch.randn(B, Hk, ctx, D, device="cuda").bfloat16()
        vc = torch.randn(B, Hk, ctx, D, device="cuda").bfloat16()
        boundary = ctx - 1 - w0
        kv, vv = kc.transpose(1, 2), vc.transpose(1, 2)
        call = lambda exchange, **kw: backend.fused_jetlong_decode_cache(
            q, qg, kc, vc, boundary=boundary, inv_freq=inv, group_size=G, has_any_pad=False, training=False,
            exchange=exchange, **kw)
        variants = []
        if shard is None:
            segs = [ops.KvSegment(kv[:, :boundary], vv[:, :boundary], 1), ops.KvSegment(kv[:, boundary:], vv[:, boundary:], 0)]
            variants.append(("pregrouped", lambda: ops.decode_segments([q, qg], segs, return_lse=False)))
            variants.append(("inplace_regroup", lambda: call(None)))
        else:
            # sharded: every rank streams its contiguous range (kc doubles as the regrouped cache: same bytes moved);
            # the partials cross NVLink through jl_peer_merge if every rank can set it up AND it reproduces the
            # NCCL all-gather + jl_merge result here, else through NCCL
            exch = "nccl"
            try:
                ok = int(torch.equal(call("peer"), call("nccl")))
            except Exception:
                ok = 0
            agree = torch.tensor([ok], device="cuda")
            torch.distributed.all_reduce(agree, op=torch.distributed.ReduceOp.MIN)
            if int(agree) == 1:
                exch = "peer"
            exchange_used[f"batch{B}"] = exch
            variants.append(("pregrouped", lambda e: call(e, key_cache_group=kc), exch))
            variants.append(("inplace_regroup", lambda e: call(e), exch))
            if exch == "peer":
                variants.append(("pregrouped_nccl_exchange", lambda e: call(e, key_cache_group=kc), "nccl"))

        def measure(fn):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            graph = None
            try:                                   # kernels + (for N > 1) the exchange in one graph
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    fn()
                graph.replay()
                torch.cuda.synchronize()
            except Exception:
                if shard is None:
                    raise
                graph = None
                torch.cuda.synchronize()
            ts = []
            for _ in range(iters):
                cold_l2()
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                if shard is not None:
                    torch.distributed.barrier()
                s.record()
                graph.replay() if graph is not None else fn()
                e.record()
                torch.cuda.synchronize()
                ts.append(s.elapsed_time(e) * 1e3)
            us = statistics.median(ts)
            if shard is not None:
                t = torch.tensor([us], device="cuda")
                torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
                us = float(t)
            return us

        def peer_wait_gave_up():
            """True on every rank if a bounded wait of jl_peer_merge ran out on any rank (the status words are cleared)."""
            st = ops.kernel_status()
            bad = torch.tensor([int(st["peer_exchange_failed"])], device="cuda")
            torch.distributed.all_reduce(bad, op=torch.distributed.ReduceOp.MAX)
            if int(bad):
                ops.clear_peer_status()
            return bool(int(bad))

        res = {}
        for tag, fn, *how in variants:
            if fn is None or (variants_wanted is not None and tag not in variants_wanted):
                continue
            if shard is None:
                us = measure(fn)
            else:
                us = measure(lambda: fn(how[0]))
                if how[0] == "peer" and peer_wait_gave_up():       # never report a number whose exchange timed out
                    us = measure(lambda: fn("nccl"))
                    exchange_used[f"batch{B}"] = "nccl"
            nbytes = B * ctx * Hk * D * 2 * 2 / world            # K and V bytes ONE rank streams, against one GPU's peak
            res[tag] = dict(us=round(us, 2), gbs_per_gpu=round(nbytes / us / 1e3, 1),
                            frac_of_measured_hbm=round(nbytes / us / 1e3 / peaks["hbm_gbs"], 4),
                            frac_of_nominal_8tbs=round(nbytes / us / 1e3 / 8000.0, 4))
        out[f"batch{B}"] = res
        del kc, vc, kv, vv
    out["config"] = dict(heads=H, kv_heads=Hk, head_dim=D, ctx=ctx, w_0=w0, group_size=G,
                         bytes="K and V bytes one rank streams per call (batch * ctx * kv_heads * head_dim * 2 * 2 / ranks); the "
                               "denominator is a copy bandwidth, which a read-only stream can exceed by a few percent",
                         timing="CUDA graph replay" if shard is None else
                         "CUDA graph replay incl. the exchange of the partials (eager if capture fails), max over ranks",
                         exchange={k: ("jl_peer_merge over peer-mapped memory" if v == "peer" else "NCCL all-gather + jl_merge")
                                   for k, v in exchange_used.items()} or None,
                         l2="256 MB write + 256 MB read before every iteration (cold, clean L2)")
    return out


# --------------------------------------------------------------------------------------------------
# instrumentation: launches that go through the C ABI are counted here, not in the product modules
# --------------------------------------------------------------------------------------------------

class LaunchCounter:
    """Wraps the kernel-launching entry points of the loaded library object: counts the kernels each call
    launches and, while `sink` is a list, brackets every jl_prefill call with a CUDA event pair on the stream
    the kernel is launched on."""
    KERNELS_PER_CALL = {"jl_prefill": 1, "jl_decode": 1, "jl_decode_static": 1, "jl_merge": 1, "jl_rotate": 1,
                        "jl_norm_rope": 1, "jl_rmsnorm": 1, "jl_step_advance": 1, "jl_decode_append": 1,
                        "jl_silu_mul": 1, "jl_peer_merge": 1}

    def __init__(self, lib):
        self.count, self.sink = 0, None
        for name, n in self.KERNELS_PER_CALL.items():
            setattr(lib, name, self._wrap(getattr(lib, name), name, n))

    def _wrap(self, fn, name, n):
        def call(*a):
            self.count += n
            if self.sink is None or name != "jl_prefill":
                return fn(*a)
            stream = torch.cuda.current_stream()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(stream)
            rc = fn(*a)
            e.record(stream)
            self.sink.append((s, e))
            return rc
        return call


def profiled_traffic_bytes(seq: int):
    """DRAM read + write bytes of one jl_prefill launch, from the committed ncu summary of the 32768-token case
    (profiles/), scaled by tokens: every operand crosses HBM once and K/V re-reads are L2 hits, so traffic grows
    in proportion to the sequence length.  None if the summary is missing."""
    import re
    path = os.path.join(ROOT, "profiles", "prefill_tc_kernel__qwen3-8b_1layer_32k.md")
    try:
        text = open(path).read()
        rd = re.search(r"dram__bytes_read\.sum`?\s*\|\s*([0-9.]+)\s*MB", text)
        wr = re.search(r"dram__bytes_write\.sum`?\s*\|\s*([0-9.]+)\s*MB", text)
        return round((float(rd.group(1)) + float(wr.group(1))) * 1e6 * seq / 32768)
    except (OSError, AttributeError, ValueError):
        return None


SP_BLOCK = 256       # tokens per placement block of the sequence-parallel runs (a multiple of the 256 query rows of a CTA)


@torch.inference_mode()
def sharded_parity(shard):
    """One layer's token-sharded attention, both exchanges, on a 4 x world x 1024-token case against the same
    rank's UNSHARDED kernel on the whole problem: max-abs and cosine over this rank's rows, worst rank reported."""
    import torch.distributed as dist
    from jetlm.kernels import cute_jetlong_backend as backend, jetlong_ops as ops
    world, blk = shard.world, shard.block
    S, H, Hk, D, G = 4 * world * 1024, 32, 8, 128, 4
    w0 = S // 4
    torch.manual_seed(1234)                                   # the same tensors on every rank
    inv = (1.0 / (1.0e6 ** (torch.arange(0, D, 2, device="cuda").float() / D)))
    q = torch.randn(1, S, H, D, device="cuda").bfloat16()
    k = torch.randn(1, S, Hk, D, device="cuda").bfloat16()
    v = torch.randn(1, S, Hk, D, device="cuda").bfloat16()
    ref = ops.posmap_prefill([q, ops.rope_regroup(q, inv, group_size=G)], [k, ops.rope_regroup(k, inv, group_size=G)], v,
                             pmap=ops.PositionMap.jetlong(w0), q_pos0=0, return_lse=False)
    rows = shard.owned_rows(S).cuda()
    ql, kl, vl = q[:, rows].contiguous(), k[:, rows].contiguous(), v[:, rows].contiguous()
    res = {}
    for mode in ("kv_gather", "q_exchange"):
        got = backend.fused_jetlong_prefill_token_sharded(ql, kl, None, vl, q_start=0, inv_freq=inv, group_size=G,
                                                          window_size_left=w0, softmax_scale=D ** -0.5, mode=mode)
        a, e = got.float().flatten().double(), ref[:, rows].float().flatten().double()
        stats = torch.tensor([float((a - e).abs().max()), -float((a @ e) / (a.norm() * e.norm()))], device="cuda")
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        res[mode] = dict(max_abs=round(float(stats[0]), 5), cos=round(-float(stats[1]), 7))
    res["case"] = f"{S} tokens, 32/8 heads, w_0 {w0}, G {G}, block {blk}; tolerance 2e-2 / 0.9999"
    res["ok"] = all(res[m]["max_abs"] <= 2e-2 and res[m]["cos"] >= 0.9999 for m in ("kv_gather", "q_exchange"))
    return res


# --------------------------------------------------------------------------------------------------
# the other BASELINE configurations, as numbers (N = 1 only; the default line stays the metric config)
# --------------------------------------------------------------------------------------------------

def _time_ms(fn, iters=3, warm=2):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    return statistics.median(ts)


@torch.inference_mode()
def prefill_length_sweep(model, cfg, lengths, w):
    """Full-model prefill tok/s of the resident model at shorter prompts (the reference's sweep protocol:
    scripts/throughput/bench_prefill_throughput.py:59-60), same w; w_0 = w."""
    out = {}
    gen = torch.Generator().manual_seed(2)
    for n in lengths:
        ids = torch.randint(0, cfg.vocab_size, (1, n), generator=gen).cuda()
        ms = _time_ms(lambda: model(input_ids=ids, use_cache=True, logits_to_keep=0).logits[0, -1], iters=2, warm=2)
        out[str(n)] = dict(tok_per_s=round(n / ms * 1e3, 1), ms=round(ms, 1), group_size=max(1, math.ceil(n / w)))
    return out


@torch.inference_mode()
def extra_configs(peaks, args):
    """BASELINE configs 2 and 3, the reference decode bench's other protocol points, and a same-box library anchor."""
    from jetlm.kernels import jetlong_ops as ops
    from jetlm.modeling.jetlong_fused import Qwen3JetLongFusedForCausalLM
    out = {}
    D = 128
    # config 2: Qwen3-1.7B full-model prefill, 65536 tokens, w_0 = 32768
    cfg2 = model_config("qwen3-1.7b", 32768, 32768, None)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    torch.manual_seed(0)
    with torch.device("cuda"):
        m2 = Qwen3JetLongFusedForCausalLM(cfg2).eval()
    torch.set_default_dtype(prev)
    ids = torch.randint(0, cfg2.vocab_size, (1, 65536), generator=torch.Generator().manual_seed(3)).cuda()
    lib = sys.modules["jetlm.kernels._native"].lib()
    counter = getattr(lib, "_bench_counter", None)
    if counter is not None:
        counter.sink = []
    ms = _time_ms(lambda: m2(input_ids=ids, use_cache=True, logits_to_keep=0).logits[0, -1], iters=3, warm=2)
    H2 = cfg2.num_attention_heads
    flops2 = 4.0 * D * H2 * 65536 * 65537 / 2
    attn_ms = None
    if counter is not None and counter.sink:
        torch.cuda.synchronize()
        attn_ms = statistics.mean(s.elapsed_time(e) for s, e in counter.sink)
        counter.sink = None
    out["config2_qwen3_1.7b_65536"] = dict(
        tok_per_s=round(65536 / ms * 1e3, 1), ms_per_step=round(ms, 1), layers=cfg2.num_hidden_layers, heads=H2,
        jl_prefill_mean_ms=round(attn_ms, 3) if attn_ms else None,
        jl_prefill_tflops=round(flops2 / (attn_ms * 1e-3) / 1e12, 1) if attn_ms else None,
        frac_of_sustained_bf16=round(flops2 / (attn_ms * 1e-3) / 1e12 / peaks["bf16_tflops_sustained"], 4) if attn_ms else None)
    del m2, ids
    torch.cuda.empty_cache()

    # config 3: Qwen3-4B head geometry (32 / 8 heads), 131072 tokens, three position maps through one kernel family
    S, H, Hk = 131072, 32, 8
    inv = 1.0 / (1.0e6 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    torch.manual_seed(4)
    q = torch.randn(1, S, H, D, device="cuda").bfloat16()
    k = torch.randn(1, S, Hk, D, device="cuda").bfloat16()
    v = torch.randn(1, S, Hk, D, device="cuda").bfloat16()
    flops3 = 4.0 * D * H * S * (S + 1) / 2
    maps = {}
    qb, kb = ops.rope_base(q, inv), ops.rope_base(k, inv)
    cases = {
        "jetlong_w0_32768": (ops.PositionMap.jetlong(32768), [qb, ops.rope_regroup(qb, inv, group_size=4)],
                             [kb, ops.rope_regroup(kb, inv, group_size=4)]),
        "selfext_g8_w2048": (ops.PositionMap.selfext(2048), [qb, ops.rope_rotate(q, inv, div=8, add=2048 - 2048 // 8)],
                             [kb, ops.rope_rotate(k, inv, div=8)]),
    }
    s_, w_ = 32768, 4096
    kr = ops.rope_rotate(k, inv, div_mul=0, mod=s_, mod_mul=1)
    cases["dca_chunk_32768"] = (ops.PositionMap.dca(s_),
                                [ops.rope_rotate(q, inv, div_mul=0, mod=s_, mod_mul=1),
                                 ops.rope_rotate(q, inv, div_mul=0, mod=s_, mod_mul=1, add=s_, t_max=s_ + w_),
                                 ops.rope_rotate(q, inv, div_mul=0, add=s_ + w_)], [kr, kr, kr])
    o = torch.empty_like(q)
    for name, (pm, qo, ko) in cases.items():
        ms = _time_ms(lambda: ops.posmap_prefill(qo, ko, v, pmap=pm, q_pos0=0, out=o, return_lse=False), iters=3, warm=1)
        maps[name] = dict(ms=round(ms, 2), tflops=round(flops3 / (ms * 1e-3) / 1e12, 1),
                          frac_of_burst_bf16=round(flops3 / (ms * 1e-3) / 1e12 / peaks["bf16_tflops"], 4))
        # the same launch on the CTA-pair kernel (cta_group::2, impl = 2; built, measured, not the default)
        ms2 = _time_ms(lambda: ops.posmap_prefill(qo, ko, v, pmap=pm, q_pos0=0, out=o, return_lse=False, impl=2), iters=3, warm=1)
        maps[name]["cta_pair_kernel_ms"] = round(ms2, 2)
        maps[name]["cta_pair_kernel_tflops"] = round(flops3 / (ms2 * 1e-3) / 1e12, 1)
    # north_star subsystem 1 as worded: the far class remapped inside the kernel, from the base-rotated operands alone
    pm = ops.PositionMap.jetlong(32768)
    ms = _time_ms(lambda: ops.posmap_prefill([qb], [kb], v, pmap=pm, q_pos0=0, out=o, return_lse=False, remap_far=(inv, 4)),
                  iters=2, warm=1)
    ms_pre = _time_ms(lambda: ops.posmap_prefill([qb, ops.rope_regroup(qb, inv, group_size=4)],
                                                 [kb, ops.rope_regroup(kb, inv, group_size=4)], v, pmap=pm, q_pos0=0, out=o,
                                                 return_lse=False), iters=2, warm=1)
    maps["jetlong_far_class_remapped_in_kernel"] = dict(
        ms=round(ms, 2), tflops=round(flops3 / (ms * 1e-3) / 1e12, 1),
        pre_rotated_incl_both_rotate_passes_ms=round(ms_pre, 2),
        pre_rotated_incl_both_rotate_passes_tflops=round(flops3 / (ms_pre * 1e-3) / 1e12, 1),
        note="jl_prefill with remap_far_in_kernel against the default form (two jl_rotate passes + jl_prefill); the slower one is not the default")
    out["config3_attention_131072_32x8_heads"] = dict(maps, note="one attention launch per map, kernel timed alone (burst peak); "
                                                      "operands from jl_rotate; parity of these maps at this size: tests/test_full_size_gpu.py")
    del cases, qb, kb, kr
    # same-shape library anchor: torch SDPA causal attention (flash / cuDNN backend), kv heads expanded to 32
    try:
        from torch.nn.attention import SDPBackend, sdpa_kernel
        qh = q.transpose(1, 2)
        kh = k.transpose(1, 2).repeat_interleave(H // Hk, dim=1)
        vh = v.transpose(1, 2).repeat_interleave(H // Hk, dim=1)
        with sdpa_kernel([SDPBackend.FLASH_ATTENTION, SDPBackend.CUDNN_ATTENTION, SDPBackend.EFFICIENT_ATTENTION]):
            ms = _time_ms(lambda: torch.nn.functional.scaled_dot_product_attention(qh, kh, vh, is_causal=True), iters=3, warm=1)
        out["sdpa_causal_anchor_131072_32_heads"] = dict(ms=round(ms, 2), tflops=round(flops3 / (ms * 1e-3) / 1e12, 1),
                                                         note="torch.nn.functional.scaled_dot_product_attention, plain causal mask "
                                                              "(no bifocal map): a same-box library anchor, not a component")
        del qh, kh, vh
    except Exception as err:      # backend not available for this shape on this build
        out["sdpa_causal_anchor_131072_32_heads"] = dict(error=str(err)[:200])
    del q, k, v, o
    torch.cuda.empty_cache()

    # the reference decode bench's other protocol points (scripts/throughput/bench_cute_decode_sm90_jetlong.py:166-172)
    pts = {}
    for ctx in (32769, 65537, 131073):
        for w0 in (4096, 32768):
            if ctx - 1 - w0 <= 0:
                continue
            r = decode_microbench(peaks, None, iters=10, ctx=ctx, w0=w0, batches=(1,))
            pts[f"ctx{ctx}_w0_{w0}"] = r["batch1"]
    out["decode_attn_protocol_points_b1"] = pts
    return out


# --------------------------------------------------------------------------------------------------
# main arm
# --------------------------------------------------------------------------------------------------

@torch.inference_mode()
def long_generate(args, cfg, model, shard, world):
    """Chunked prefill of a long prompt into the preallocated KV cache (every rank keeps a block-cyclic stripe
    when N > 1), then greedy one-token steps on the same cache.  Times are device times, max over ranks."""
    import torch.distributed as dist
    from jetlm.kernels.kv_cache import BifocalKVCache
    T, steps = args.long_generate, args.decode_steps
    model.model.kernels_within_window = True                  # the first chunk (L <= w) runs on the same kernels
    gen = torch.Generator().manual_seed(1)
    ids = torch.randint(0, cfg.vocab_size, (1, T), generator=gen).cuda()
    cache = BifocalKVCache(cfg, T + steps, device="cuda", dtype=torch.bfloat16, shard=shard,
                           regrouped_far_keys=args.regrouped_far_keys and not args.eager_decode)

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def device_ms(fn):
        sync()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        r = fn()
        e.record()
        sync()
        ms = torch.tensor([s.elapsed_time(e)], device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms), r

    def prefill():
        hidden = None
        for lo in range(0, T, args.chunk):
            hidden = model.model(input_ids=ids[:, lo: lo + args.chunk], past_key_values=cache, use_cache=True).last_hidden_state
        token = model.lm_head(hidden[:, -1:, :]).argmax(-1)
        if world > 1:
            dist.broadcast(token, src=world - 1)
        return token

    def decode(token):
        out = []
        if not args.eager_decode:
            from jetlm.kernels.decode_graph import GraphedDecodeStep
            step = GraphedDecodeStep(model, cache)
            step(token)                                   # captures (one eager run + capture), replays: token 1
            out.append(step.token.clone())
            sync()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(steps - 1):
                out.append(step().clone())
            e.record()
            sync()
            ms = torch.tensor([s.elapsed_time(e)], device="cuda")
            if world > 1:
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            replay_ms[0] = float(ms) / max(steps - 1, 1)
            return torch.cat(out, 1)
        for _ in range(steps):
            hidden = model.model(input_ids=token, past_key_values=cache, use_cache=True).last_hidden_state
            token = model.lm_head(hidden[:, -1:, :]).argmax(-1)
            if world > 1:
                dist.broadcast(token, src=0)
            out.append(token)
        return torch.cat(out, 1)

    replay_ms = [None]
    # warm-up on a short prompt (same code paths, allocator and NCCL set-up), then the measured run
    warm = min(T, 2 * args.chunk)
    for lo in range(0, warm, args.chunk):
        model.model(input_ids=ids[:, lo: lo + args.chunk], past_key_values=cache, use_cache=True)
    model.model(input_ids=ids[:, :1], past_key_values=cache, use_cache=True)
    cache.reset()
    pre_ms, token = device_ms(prefill)
    dec_ms, toks = device_ms(lambda: decode(token))
    layer = cache.layers[0]
    return dict(metric="long_generate", n_gpus=world, prompt_tokens=T, chunk=args.chunk, decode_steps=steps,
                prefill_s=round(pre_ms / 1e3, 3), prefill_tok_per_s=round(T / (pre_ms / 1e3), 1),
                decode_ms_per_token=round(replay_ms[0] if replay_ms[0] is not None else dec_ms / steps, 3),
                decode_tok_per_s=round(1e3 / (replay_ms[0] if replay_ms[0] is not None else dec_ms / steps), 2),
                decode_mode="one CUDA graph replay per token (capture excluded from the time)" if replay_ms[0] is not None
                else "Python-launched steps",
                group_size_at_end=max(1, math.ceil((T + steps) / args.w)),
                kv_cache_gb_per_rank=round((3 if layer.group_keys is not None else 2) * layer.keys.numel() * 2
                                           * cfg.num_hidden_layers / 1e9, 2),
                regrouped_far_keys=layer.group_keys is not None,
                kv_rows_per_rank=layer.rows, tokens_in_cache=cache.get_seq_length(),
                first_tokens=toks[0, :8].tolist(),
                config=dict(model=args.model, w=args.w, w_0=args.w0, layers=cfg.num_hidden_layers,
                            cache=f"preallocated, block-cyclic stripes of {SP_BLOCK} tokens over ranks" if world > 1 else "preallocated"))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="qwen3-8b", choices=sorted(MODEL_DIMS))
    ap.add_argument("--seq", type=int, default=131072)
    ap.add_argument("--w", type=int, default=32768)
    ap.add_argument("--w0", type=int, default=32768)
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (debug only; shown in config)")
    ap.add_argument("--logits-to-keep", type=int, default=0)
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--only-decode", action="store_true", help="run just the decode-attention microbench (profiling aid)")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the other BASELINE configurations (N = 1 only)")
    ap.add_argument("--long-generate", type=int, default=0, metavar="TOKENS",
                    help="instead of the default workload: chunked prefill of TOKENS tokens into the preallocated "
                         "(sequence-sharded when N > 1) KV cache, then --decode-steps greedy tokens")
    ap.add_argument("--chunk", type=int, default=32768)
    ap.add_argument("--decode-steps", type=int, default=256)
    ap.add_argument("--regrouped-far-keys", action="store_true", help="--long-generate: keep regrouped copies of the far "
                    "keys in a second cache buffer (+50 %% KV memory) so decode streams them as stored")
    ap.add_argument("--eager-decode", action="store_true", help="--long-generate: launch every decode step from Python "
                    "instead of replaying one CUDA graph per token")
    args = ap.parse_args()

    if args.impl == "reference":
        run_reference(args)
        return

    from jetlm.kernels import _native
    counter = LaunchCounter(_native.lib())            # fails loudly right away if the extension is missing
    _native.lib()._bench_counter = counter
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU path")

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    shard = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        from jetlm.kernels import cute_jetlong_backend as backend
        from jetlm.kernels.sequence_parallel import SequenceShard
        shard = SequenceShard(rank, world, block=SP_BLOCK)
        backend.configure_sequence_sharding(shard)

    from jetlm.kernels import jetlong_ops as ops
    from jetlm.modeling.jetlong_fused import Qwen3JetLongFusedForCausalLM

    peaks = load_peaks()
    if args.only_decode:
        res = decode_microbench(peaks, shard, iters=max(args.steps, 1))
        if rank == 0:
            print(json.dumps(dict(metric="decode_attn_us", unit="us", n_gpus=world, decode_attn=res)), flush=True)
        if world > 1:
            torch.distributed.destroy_process_group()
        return
    cfg = model_config(args.model, args.w, args.w0, args.layers or None)
    G = max(1, math.ceil(args.seq / args.w))
    torch.manual_seed(0)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    with torch.device("cuda"):
        model = Qwen3JetLongFusedForCausalLM(cfg).eval()
    torch.set_default_dtype(prev)
    if shard is not None:
        # sequence parallel: every rank embeds / projects / stores only its block-cyclic stripe of the prompt
        model.model.token_sharded = True

    if args.long_generate:
        line = long_generate(args, cfg, model, shard, world)
        if rank == 0:
            print(json.dumps(line), flush=True)
        if world > 1:
            torch.distributed.destroy_process_group()
        return

    gen = torch.Generator().manual_seed(1)
    ids_host = torch.randint(0, cfg.vocab_size, (1, args.seq), generator=gen).pin_memory()
    ids_dev = ids_host.cuda()
    result_host = torch.empty(cfg.vocab_size, dtype=torch.bfloat16).pin_memory()

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    @torch.inference_mode()
    def step(ids):
        out = model(input_ids=ids, use_cache=True, logits_to_keep=args.logits_to_keep)
        return out.logits[0, -1]

    @torch.inference_mode()
    def step_e2e():
        ids = ids_host.to("cuda", non_blocking=True)
        last = step(ids)
        result_host.copy_(last, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def timed(fn, k):
        barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(k):
            fn()
        e.record()
        barrier()
        ms = torch.tensor([s.elapsed_time(e)], device="cuda")
        if world > 1:
            torch.distributed.all_reduce(ms, op=torch.distributed.ReduceOp.MAX)
        return float(ms)

    parity = sharded_parity(shard) if shard is not None else None
    if parity is not None and not parity["ok"]:
        raise RuntimeError(f"sharded attention does not reproduce the unsharded kernel: {parity}")

    for _ in range(args.warmup):
        step(ids_dev)
    launches0 = counter.count
    sampler = ClockSampler(local)
    sampler.start()
    counter.sink = sink = []
    total_ms = timed(lambda: step(ids_dev), args.steps)
    counter.sink = None
    launches = counter.count - launches0
    e2e_ms = timed(step_e2e, args.steps)
    clocks = sampler.stop()
    status = ops.kernel_status()                      # the bounded waits of the kernels: a timeout invalidates the numbers
    if status["prefill_wait_timeouts"] or status["peer_exchange_failed"]:
        raise RuntimeError(f"a bounded wait inside the kernels gave up during the timed region: {status}")
    sp_mode = None
    if shard is not None:
        from jetlm.kernels import cute_jetlong_backend as backend
        sp_mode = backend.LAST_TOKEN_SHARDED_MODE

    # roofline of the dominant kernel: algorithmic FLOPs of one launch / its mean device time
    torch.cuda.synchronize()
    pre = [s_.elapsed_time(e_) for s_, e_ in sink]
    H, D = cfg.num_attention_heads, 128
    # per layer and rank: one launch over the rank's query stripe and all keys (K/V gather), or N launches, one per
    # query stripe against the local key stripe (Q exchange)
    flops_launch = 4.0 * D * H * args.seq * (args.seq + 1) / 2 / (world if sp_mode == "kv_gather" else world ** 2)
    mean_ms = statistics.mean(pre) if pre else float("nan")
    achieved = flops_launch / (mean_ms * 1e-3) / 1e12
    roofline = dict(bound="tensor", kernel="jl_prefill (bifocal attention)", achieved=round(achieved, 1),
                    peak=peaks["bf16_tflops_sustained"], unit="TFLOP/s",
                    frac=round(achieved / peaks["bf16_tflops_sustained"], 4), peak_source=peaks["source"] + " (sustained)",
                    frac_of_burst=round(achieved / peaks["bf16_tflops"], 4), frac_of_nominal_2250=round(achieved / 2250.0, 4),
                    launches_timed=len(pre), mean_launch_ms=round(mean_ms, 3),
                    attention_share_of_step=round(sum(pre) / total_ms, 4) if pre else None,
                    algorithmic_flops_per_launch=flops_launch,
                    traffic=profiled_traffic_bytes(args.seq) if world == 1 else None,
                    traffic_source="profiles/prefill_tc_kernel__qwen3-8b_1layer_32k.md (ncu, 32768 tokens), scaled by tokens"
                    if world == 1 else "not captured for the sharded launches")

    line = dict(metric="prefill_tok_per_s", value=round(args.seq * args.steps / (total_ms * 1e-3), 1), unit="tok/s",
                n_gpus=world, steps=args.steps, warmup=args.warmup, ms_per_step=round(total_ms / args.steps, 2),
                higher_is_better=True, scaling="strong", vs_baseline=None, dtype="bf16", data="synthetic",
                config=workload_config(args, cfg, G, sp_mode), clocks=clocks,
                e2e=dict(value=round(args.seq * args.steps / (e2e_ms * 1e-3), 1), unit="tok/s",
                         h2d_bytes_per_step=ids_host.numel() * ids_host.element_size(),
                         d2h_bytes_per_step=result_host.numel() * result_host.element_size()),
                gpu_launches=launches, roofline=roofline, kernel_status=status)
    if parity is not None:
        line["sharded_parity"] = parity
    if world == 1 and not args.no_extras and args.seq == 131072 and args.model == "qwen3-8b" and not args.layers:
        line["prefill_length_sweep"] = prefill_length_sweep(model, cfg, (32768, 65536), args.w)

    del model
    torch.cuda.empty_cache()
    if not args.no_decode:
        line["decode_attn"] = decode_microbench(peaks, shard)
        ops.check_status()
    if world == 1 and not args.no_extras:
        line["other_configs"] = extra_configs(peaks, args)
    if rank == 0 and world == 1 and not args.no_cpu:
        c = cpu_prefill_sample(args.seq, model_dims(cfg), args.w0, G)
        line["cpu_baseline"] = dict(value=round(c["tok_s"], 3), unit="tok/s", cores=c["cores"], kind="port", sample=c["sample"],
                                    sample_seconds=round(c["sample_s"], 2))
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
