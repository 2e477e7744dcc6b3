#!/usr/bin/env python
"""Benchmark of the sm_100a hot path. Prints ONE JSON line (rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload llama|nanogpt|gemm|attention]
    python bench.py --impl reference ...      # the CPU baseline arm on the host cores

Workloads (synthetic, seeded; shapes of the five benchmark configurations):
  llama      (default) Llama-style decoder stack forward, bf16, 8 layers, d 4096, 32/8 heads,
             FFN 14336, seq 4096, batch 4; tensor-parallel over the N GPUs (strong scaling);
             metric = forward tokens/s. The line also carries the GEMM and attention kernel
             throughputs measured in the same process at N=1 (`kernels`).
  nanogpt    nanoGPT forward, 12 layers, d 768, seq 1024, batch 16, vocab 50304; TP up to 4,
             8 GPUs = TP4 x 2 batch halves.
  gemm       bf16 GEMM + bias + ReLU, M=N=K=4096 (`--k` for the K sweep); TFLOP/s.
  attention  flash attention forward, B8 H16 S2048 D128 (`--causal`); TFLOP/s.

`value` is measured with inputs resident in HBM; `e2e` is the same metric through host
buffers: every step copies the inputs from pinned host memory and reads the result back.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PEAKS_FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(PEAKS_FALLBACK), "fallback"


class ClockSampler:
    """Samples SM clock, power and throttle reasons of one GPU with nvidia-smi while the
    timed region runs."""

    FIELDS = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        fd, self.path = tempfile.mkstemp(suffix=".csv")
        os.close(fd)
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL,
            )
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, reasons, max_mhz, power = [], set(), None, []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 7:
                    continue
                try:
                    clocks.append(float(parts[0]))
                    max_mhz = float(parts[1])
                    power.append(float(parts[2]))
                except ValueError:
                    continue
                for name, val in zip(names, parts[3:7]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        os.remove(self.path)
        if clocks:
            # the busiest half of the samples: the sampler also sees the gaps between loops
            busy = sorted(zip(power, clocks))[len(clocks) // 2 :]
            out.update(sm_mhz=statistics.median(c for _, c in busy), sm_max_mhz=max_mhz, reasons=sorted(reasons), samples=len(clocks), power_w_max=max(power))
        return out


class Dist:
    """torch.distributed plumbing: rendezvous, barrier, max over ranks, NCCL ids for groups."""

    def __init__(self, n_gpus: int):
        import torch

        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != n_gpus and self.world > 1:
            raise SystemExit(f"--gpus {n_gpus} but WORLD_SIZE={self.world}")
        if n_gpus > 1 and self.world == 1:
            raise SystemExit("for --gpus N > 1 launch with: python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 bench.py --gpus N ...")
        torch.cuda.set_device(self.local_rank)
        if self.world > 1:
            import torch.distributed as dist

            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))
            self.dist = dist
        else:
            self.dist = None

    def barrier(self):
        import torch

        torch.cuda.synchronize()
        if self.dist:
            self.dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(self, value: float) -> float:
        if not self.dist:
            return value
        import torch

        t = torch.tensor([value], device="cuda", dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(self, value: float) -> float:
        if not self.dist:
            return value
        import torch

        t = torch.tensor([value], device="cuda", dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return float(t.item())

    def group_unique_id(self, group_leader: int, nccl_path):
        """Every group leader creates an NCCL id; all ranks receive their leader's."""
        from lighthouse_b200.context import nccl_unique_id

        mine = nccl_unique_id(nccl_path) if self.rank == group_leader else None
        ids = [None] * self.world
        self.dist.all_gather_object(ids, mine)
        return ids[group_leader]

    def close(self):
        if self.dist:
            self.dist.destroy_process_group()


def timed_loop(dist: Dist, stream, step, steps: int, warmup: int, before_end=None):
    """W untimed steps, then exactly K steps between a barrier + synchronize on both sides,
    timed with CUDA events on the launching stream; returns the max over ranks in ms.
    ``before_end`` makes the launching stream wait for work the steps put on other streams, so
    that the closing event covers it."""
    import torch

    for _ in range(warmup):
        step()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        step()
    if before_end is not None:
        before_end()
    e1.record(stream)
    stream.synchronize()
    dist.barrier()
    return dist.max_over_ranks(e0.elapsed_time(e1))


def gemm_roofline(plan, op_ms, peaks, which):
    """Roofline entry for the dominant kernel of a decoder step: all GEMM launches of one
    step, algorithmic 2MNK flops over their CUDA-event durations."""
    flops = sum(op.flops() for op in plan.ops if op.kind in ("gemm", "gemm_rope"))
    ms = float(sum(t for op, t in zip(plan.ops, op_ms) if op.kind in ("gemm", "gemm_rope")))
    achieved = flops / (ms * 1e-3) / 1e12 if ms > 0 else 0.0
    peak = peaks["bf16_tflops_sustained"]
    share = {}  # with the overlapped schedule the side-stream operators' spans overlap the others'
    for op, t in zip(plan.ops, op_ms):
        if op.kind not in ("stream", "event_record", "event_wait", "reserve_sms"):
            share[op.kind] = share.get(op.kind, 0.0) + max(float(t), 0.0)
    total = sum(share.values()) or 1.0
    return {
        "bound": "tensor", "kernel": "gemm_bf16_tc_kernel", "achieved": round(achieved, 1), "peak": peak, "unit": "TFLOP/s",
        "frac": round(achieved / peak, 4), "peak_source": f"{which} cuBLAS bf16, sustained (kernel timed inside a long step)", "traffic": None,
        "launches_per_step": sum(1 for op in plan.ops if op.kind in ("gemm", "gemm_rope")),
        "step_time_share": {k: round(v / total, 4) for k, v in sorted(share.items())},
    }


def decoder_parity(which: str, cfg, w, host_in, dev_out, tp_rank: int, tp: int) -> dict:
    """Outside the timed region: the result of the last step, at full depth and full size, on
    the first 256 positions of two sequences, against the CPU oracle run on those prefixes
    alone (a causal decoder's prefix depends on nothing after it)."""
    import torch

    from oracle import prefix as P
    from oracle.check import parity_report

    torch.cuda.synchronize()
    seqs, prefix = (0, cfg.batch - 1), 256
    rows = torch.from_numpy(P.prefix_rows(cfg.seq, seqs, prefix)).to(dev_out.device)
    got = dev_out[rows].float().cpu().numpy()
    if which == "llama":
        ref = P.llama_prefix_reference(w, host_in, cfg, seqs, prefix, shards=tp)
    else:
        vl = cfg.vocab // tp
        ref = P.nanogpt_prefix_reference(w, host_in, cfg, seqs, prefix, vocab_slice=slice(tp_rank * vl, (tp_rank + 1) * vl))
    from oracle.check import LAYER_ROUNDINGS, SHARDED_LAYER_ROUNDINGS

    rep = parity_report(got, ref, "bf16", n_layer=cfg.n_layer, roundings_per_layer=SHARDED_LAYER_ROUNDINGS if which == "llama" and tp > 1 else LAYER_ROUNDINGS)
    rep.update(checked="positions 0..255 of sequences %d and %d of rank 0's result at full depth vs the CPU oracle on those prefixes" % seqs
               + (" (the oracle rounds the %d devices' partial sums of each contracting product as the devices do)" % tp if which == "llama" and tp > 1 else ""),
               max_rel_err=float("%.3e" % rep["max_rel_err"]), elementwise_excess=round(rep["elementwise_excess"], 3))
    return rep


# ------------------------------------------------------------------------------- decoders
def run_decoder(args, dist: Dist, which: str) -> dict:
    import torch

    from lighthouse_b200.context import CudaContext, find_torch_nccl
    from lighthouse_b200.workloads import decoder as D
    from lighthouse_b200.workloads.session import PlanSession
    from lighthouse_b200.workloads import synthetic as I

    n = dist.world
    if which == "llama":
        cfg = D.LlamaConfig(n_layer=args.layers or 8)
        tp, dp = n, 1
    else:
        cfg = D.NanoGptConfig(n_layer=args.layers or 12)
        if args.nanogpt_layout == "dp":
            # the 16 sequences are split over the ranks: a forward pass then needs no exchange at
            # all (at d_model 768 the all-reduce of the f32 residual costs more than it saves)
            if cfg.batch % n:
                raise SystemExit(f"batch {cfg.batch} does not split over {n} GPUs")
            tp, dp = 1, n
        else:
            tp = n if n <= 4 else 4  # 12 heads do not split 8 ways: 8 GPUs = TP4 x 2 batch halves
            dp = n // tp
        cfg = D.NanoGptConfig(n_layer=cfg.n_layer, batch=cfg.batch // dp)
    D.check_tp(cfg, tp)
    tp_rank, group = dist.rank % tp, dist.rank // tp
    stream = torch.cuda.Stream()
    ctx = CudaContext(dist.local_rank)
    with torch.cuda.stream(stream):
        ctx.use_torch_stream()
    if tp > 1:
        nccl = find_torch_nccl()
        uid = dist.group_unique_id(group * tp, nccl)
        ctx.comm_init(uid, tp_rank, tp, nccl)

    # same seed on every rank, sliced locally: tp = n computes what tp = 1 computes
    if which == "llama":
        w = I.llama_weights(cfg.n_layer, cfg.dim, cfg.n_heads, cfg.n_kv_heads, cfg.ffn, seed=5)
        weights = [t.cuda() for t in D.flatten_llama_args(D.shard_llama_weights(w, cfg, tp_rank, tp))]
        overlapped = tp > 1 and args.microbatches > 0
        fused = overlapped and args.collectives == "fused"
        if fused:
            # symmetric (multicast) buffers for the fused kernel; every rank must get them, or
            # all ranks take the NCCL schedule together
            from lighthouse_b200.workloads.symmetric import SymmetricBuffers

            try:
                symm = SymmetricBuffers(ctx)
                symm_args = [symm.empty(shape, torch.bfloat16) for shape in D.llama_symmetric_args(cfg, args.microbatches)]
                failed = 0.0
            except Exception as e:  # noqa: BLE001 - reported below, never silent
                print(f"[bench] rank {dist.rank}: symmetric memory unavailable ({e}); NCCL schedule instead", file=sys.stderr)
                failed = 1.0
            if dist.sum_over_ranks(failed) > 0:
                fused = False
            else:
                weights += symm_args
        # with the fused kernel the result buffers are symmetric memory too: the last layer's
        # kernel gathers straight into them (every rank holds the whole result either way)
        plan = D.build_llama_plan_overlapped(cfg, tp_rank, tp, args.microbatches, args.reserve_sms, fused=fused, result_symmetric=fused) if overlapped else D.build_llama_plan(cfg, tp_rank, tp)
        host_in = torch.randn(cfg.tokens, cfg.dim, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16).pin_memory()
        dev_in = host_in.cuda()
        new_result = (lambda: symm.empty((cfg.tokens, cfg.dim), torch.bfloat16)) if fused else (lambda: torch.empty(cfg.tokens, cfg.dim, device="cuda", dtype=torch.bfloat16))
        dev_out = new_result()
    else:
        w = I.nanogpt_weights(cfg.n_layer, cfg.n_embd, cfg.hidden, cfg.vocab, cfg.block_size, seed=4)
        # nanoGPT has no fused collective kernel (LayerNorm, f32 residual); its overlapped schedule
        # runs on NCCL reduce-scatter / all-gather and is chosen with --collectives nccl
        fused = False
        overlapped = tp > 1 and args.microbatches > 0 and args.collectives == "nccl" and (cfg.batch // args.microbatches) % tp == 0
        weights = [t.cuda() for t in D.flatten_nanogpt_args(D.shard_nanogpt_weights(w, cfg, tp_rank, tp, full_bias=overlapped))]
        plan = D.build_nanogpt_plan_overlapped(cfg, tp_rank, tp, args.microbatches, args.reserve_sms) if overlapped else D.build_nanogpt_plan(cfg, tp_rank, tp)
        ids = torch.randint(0, cfg.vocab, (cfg.tokens * dp,), generator=torch.Generator().manual_seed(1)).to(torch.int32)
        host_in = ids[group * cfg.tokens : (group + 1) * cfg.tokens].contiguous().pin_memory()
        dev_in = host_in.cuda()
        dev_out = torch.empty(cfg.tokens, cfg.vocab // tp, device="cuda", dtype=torch.float32)
    host_out = torch.empty(dev_out.shape, dtype=dev_out.dtype).pin_memory()
    sess = PlanSession(plan, ctx=ctx)
    dev_args = [dev_out, dev_in] + weights
    total_tokens = cfg.tokens * dp

    sampler = ClockSampler(dist.local_rank)
    launches0 = ctx.launch_count
    with torch.cuda.stream(stream):
        sess.set_profiling(True)
        sampler.start()
        ms = timed_loop(dist, stream, lambda: sess.run(dev_args), args.steps, args.warmup)
        launches = (ctx.launch_count - launches0) * args.steps // (args.steps + args.warmup)
        op_ms = sess.op_times_ms()  # per-operator durations of the last timed step
        if args.timeline and dist.rank == 0:
            with open(args.timeline, "w") as f:
                for kind, strm, t0, t1 in sess.timeline_ms():
                    f.write(f"{kind:14s} stream {strm}  {t0:9.3f} -> {t1:9.3f} ms  ({t1 - t0:7.3f})\n")
        sess.set_profiling(False)

        # End to end: host -> device copy of the step's input, the step, device -> host read of
        # the result. In the overlapped schedules a rank reads only its own rows of the input
        # (the residual stream is sharded by rows) and every rank ends up with the whole
        # result, so each copies its own rows in and reads its own rows back: together the
        # ranks move the input and the result exactly once.
        if overlapped and which == "llama":
            tm = cfg.tokens // args.microbatches
            ts = tm // tp
            my_rows = [slice(mb * tm + tp_rank * ts, mb * tm + (tp_rank + 1) * ts) for mb in range(args.microbatches)]
        else:
            my_rows = None

        # Steps are pipelined the way a serving loop would: two input and two result buffers, the
        # copy of step i+1's input and the read-back of step i-1's result run on copy streams
        # under step i's kernels. Every step still moves its own input and its own result.
        dev_in2, dev_out2 = torch.empty_like(dev_in), (new_result() if which == "llama" else torch.empty_like(dev_out))
        bufs = [(dev_in, dev_out, dev_args), (dev_in2, dev_out2, [dev_out2, dev_in2] + weights)]
        h2d_stream, d2h_stream = torch.cuda.Stream(), torch.cuda.Stream()
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_done = [torch.cuda.Event() for _ in range(2)]
        ev_read = [torch.cuda.Event() for _ in range(2)]
        state = {"i": 0}
        reads_result = bool(my_rows) or dist.rank % tp == 0 or which == "nanogpt"

        def e2e_step():
            b = state["i"] & 1
            state["i"] += 1
            d_in, d_out, d_args = bufs[b]
            h2d_stream.wait_event(ev_done[b])  # the step that last read this input buffer
            with torch.cuda.stream(h2d_stream):
                if my_rows:
                    for rows in my_rows:
                        d_in[rows].copy_(host_in[rows], non_blocking=True)
                else:
                    d_in.copy_(host_in, non_blocking=True)
                ev_in[b].record(h2d_stream)
            stream.wait_event(ev_in[b])
            stream.wait_event(ev_read[b])  # the read-back that last used this result buffer
            sess.run(d_args)
            ev_done[b].record(stream)
            d2h_stream.wait_event(ev_done[b])
            with torch.cuda.stream(d2h_stream):
                if my_rows:
                    for rows in my_rows:
                        host_out[rows].copy_(d_out[rows], non_blocking=True)
                elif reads_result:
                    host_out.copy_(d_out, non_blocking=True)
                ev_read[b].record(d2h_stream)

        def e2e_loop_end():
            stream.wait_event(ev_read[0])
            stream.wait_event(ev_read[1])

        for e in ev_done + ev_read:
            e.record(stream)
        ms_e2e = timed_loop(dist, stream, e2e_step, args.steps, max(1, args.warmup // 2), before_end=e2e_loop_end)
        clocks = sampler.stop()
    ctx.sync()  # raises if any kernel gave up on a bounded wait
    parity = decoder_parity(which, cfg, w, host_in, dev_out, tp_rank, tp) if dist.rank == 0 and not args.no_parity else None
    del w
    if my_rows:
        h2d = d2h = sum(r.stop - r.start for r in my_rows) * host_in.shape[1] * host_in.element_size()
    else:
        h2d = host_in.numel() * host_in.element_size()
        d2h = host_out.numel() * host_out.element_size() if (dist.rank % tp == 0 or which == "nanogpt") else 0
    h2d_total, d2h_total = dist.sum_over_ranks(h2d), dist.sum_over_ranks(d2h)
    peaks, source = load_peaks()
    flops = cfg.flops_per_token() * total_tokens
    step_s = ms / args.steps * 1e-3
    res = {
        "metric": f"{which}_decoder_forward_tokens_per_s", "value": round(total_tokens / step_s, 1), "unit": "tokens/s",
        "n_gpus": n, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {
            "workload": workload_description(args),
            "parallelism": (f"dp{dp}: {cfg.batch} of {cfg.batch * dp} sequences per GPU, no collective in the forward pass" if (tp == 1 and dp > 1) else f"tp{tp}" + (f"xdp{dp}" if dp > 1 else "")) + (f", {'fused multimem reduce+norm+gather kernel' if fused else 'NCCL reduce-scatter/all-gather'} of {args.microbatches} micro-batches overlapped with compute" if overlapped else ""), "tokens_per_step": total_tokens, "l2": "inputs_exceed_l2 (weights + activations >> 126 MB)",
            "algorithmic_tflop_per_step": round(flops / 1e12, 3),
        },
        "model_tflops": round(flops / step_s / 1e12, 1), "model_frac_of_peak": round(flops / step_s / 1e12 / (n * peaks["bf16_tflops_sustained"]), 4),
        "roofline": gemm_roofline(plan, op_ms, peaks, source),
        "e2e": {"value": round(total_tokens / (ms_e2e / args.steps * 1e-3), 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d_total), "d2h_bytes_per_step": int(d2h_total)},
        "gpu_launches": int(launches), "clocks": clocks,
    }
    if parity is not None:
        res["parity"] = parity
    if which == "llama":
        per_layer = NCU_TRAFFIC_BYTES.get("llama_gemms_per_layer")
        res["roofline"]["traffic"] = per_layer * cfg.n_layer if (n == 1 and per_layer) else None
    sess.close()
    if fused:
        symm.close()
    ctx.close()
    return res


# ---------------------------------------------------------------------------- single kernels
# dram__bytes_read.sum + dram__bytes_write.sum per launch, measured once per kernel with
# `ncu --clock-control none -k regex:<kernel> -c 2..8` on this file's own workloads (the GEMM
# and attention workloads as they are; the decoder's GEMM launches on a 2-layer stack, summed
# per layer and multiplied by the layer count, traffic being the same for every layer).
NCU_TRAFFIC_BYTES = {"gemm_4096": 83.7e6, "attention_full": 244.8e6, "attention_causal": 561.4e6, "llama_gemms_per_layer": 5.158e9}
# The f32 GEMM runs as six bf16 products per f32 product (each operand split into three bf16
# terms): its ceiling is a sixth of the measured bf16 peak.
F32_VIA_SIX_BF16_FRACTION_OF_BF16 = 1.0 / 6.0


L2_BYTES = 126 << 20


def rotating_sets(make_set, bytes_per_set: int) -> list:
    """Copies of a kernel's operands on the device, enough of them that a set has left the L2
    (three times its capacity has gone through) before its turn comes again."""
    n = max(2, -(-3 * L2_BYTES // max(bytes_per_set, 1)))
    return [make_set() for _ in range(n)]


def time_rotating(ctx, sess, arg_sets, steps: int, warmup: int, groups: int = 5):
    """Seconds per launch: ``groups`` CUDA-event pairs on the context's stream, each around
    ``steps`` launches issued back to back, each launch on the next operand set (inputs larger
    than L2 in aggregate: every launch finds its operands in HBM, and no flush kernel leaves the
    cache full of dirty lines for the timed kernel to write back). One array entry per group:
    its elapsed time / ``steps``, so the gaps between consecutive launches are inside the figure
    and the cost of recording an event (microseconds, as much as a small kernel) is not."""
    import numpy as np
    import torch

    stream = torch.cuda.ExternalStream(ctx.stream_handle())
    torch.cuda.synchronize()
    n = len(arg_sets)
    for i in range(warmup):
        sess.run(arg_sets[i % n])
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(groups)]
    i = warmup
    for e0, e1 in pairs:
        e0.record(stream)
        for _ in range(steps):
            sess.run(arg_sets[i % n])
            i += 1
        e1.record(stream)
    ctx.sync()
    return np.array([e0.elapsed_time(e1) * 1e-3 / steps for e0, e1 in pairs])


L2_NOTE = "operand sets rotate (3 x L2 in aggregate): every timed launch reads its operands from HBM; launches back to back, one event pair per group of launches"


def kernel_gemm(ctx, peaks, source, K=4096, steps=20, warmup=5) -> dict:
    """bf16 GEMM + bias + ReLU, M = N = 4096 (config 2): one launch per step on rotating
    operand sets, one CUDA-event pair per launch."""
    import torch

    from lighthouse_b200.plan import ArgSpec, Plan
    from lighthouse_b200.workloads import synthetic as I
    from lighthouse_b200.workloads.session import PlanSession

    M = N = 4096
    a, b, bias = I.gemm_bf16_normal(M, N, K, seed=2)
    plan = Plan("gemm_bias_relu", [ArgSpec((M, N), "bf16", "d"), ArgSpec((M, K), "bf16", "a"), ArgSpec((K, N), "bf16", "b"), ArgSpec((N,), "bf16", "bias")])
    plan.gemm(plan.arg(0), plan.arg(1), plan.arg(2), bias=plan.arg(3), act="relu")
    sess = PlanSession(plan, ctx=ctx)
    sets = rotating_sets(lambda: [torch.empty(M, N, device="cuda", dtype=torch.bfloat16), a.cuda(), b.cuda(), bias.cuda()], 2 * (M * K + K * N + M * N))
    d = sets[0][0]
    times = time_rotating(ctx, sess, sets, steps, warmup)
    # the same launches as programmatic dependents of one another (a context option, off by
    # default: it hides a launch's set-up under its predecessor's tail when kernels queue back to
    # back like here, and costs end-to-end rate where other streams' copies interleave)
    ctx.set_launch_overlap(True)
    overlapped = time_rotating(ctx, sess, sets, steps, warmup)
    ctx.set_launch_overlap(False)
    sess.close()
    flops = 2.0 * M * N * K
    mean_s = float(times.mean())
    achieved = flops / mean_s / 1e12
    ov_s = float(overlapped.mean())
    return {
        "ms": round(mean_s * 1e3, 5), "best_ms": round(float(times.min()) * 1e3, 5), "tflops": round(achieved, 1), "shape": [M, N, K],
        "with_launch_overlap": {"ms": round(ov_s * 1e3, 5), "tflops": round(flops / ov_s / 1e12, 1), "frac": round(flops / ov_s / 1e12 / peaks["bf16_tflops"], 4)},
        "roofline": {"bound": "tensor", "kernel": "gemm_bf16_tc_kernel", "achieved": round(achieved, 1), "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": round(achieved / peaks["bf16_tflops"], 4), "peak_source": f"{source} cuBLAS bf16, burst (kernel timed alone)", "traffic": NCU_TRAFFIC_BYTES["gemm_4096"] if K == 4096 else None},
        "host": (a, b, bias, d),
    }


def kernel_gemm_f32(ctx, peaks, source, steps=20, warmup=5) -> dict:
    """f32 GEMM accumulating into C, M = N = K = 1024, A, B ~ U(-1, 1) (config 1): the lh-run
    matmul. Runs as six bf16 products on the tensor cores (one operand-split launch + one
    tcgen05 GEMM whose stages hold the three bf16 terms of both operands, four accumulators per
    tile); the flop count is the f32 problem's 2MNK."""
    import torch

    from lighthouse_b200.plan import ArgSpec, Plan
    from lighthouse_b200.workloads import synthetic as I
    from lighthouse_b200.workloads.session import PlanSession

    M = N = K = 1024
    a, b, c = I.gemm_f32_uniform(M, N, K, seed=1)
    plan = Plan("matmul_f32", [ArgSpec((M, K), "f32", "a"), ArgSpec((K, N), "f32", "b"), ArgSpec((M, N), "f32", "c")])
    plan.gemm(plan.arg(2), plan.arg(0), plan.arg(1), c=plan.arg(2))
    sess = PlanSession(plan, ctx=ctx)
    sets = rotating_sets(lambda: [torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda(), torch.from_numpy(c).cuda()], 4 * (M * K + K * N + M * N))
    times = time_rotating(ctx, sess, sets, steps, warmup)
    sess.close()
    mean_s = float(times.mean())
    achieved = 2.0 * M * N * K / mean_s / 1e12
    peak = peaks["bf16_tflops"] * F32_VIA_SIX_BF16_FRACTION_OF_BF16
    return {"ms": round(mean_s * 1e3, 5), "best_ms": round(float(times.min()) * 1e3, 5), "tflops": round(achieved, 2), "shape": [M, N, K],
            "path": "six bf16 products (operands split in three bf16 terms) on tcgen05, two launches; f32 result within 1e-5 of the loop nest",
            "roofline": {"bound": "tensor", "kernel": "split_bf16x3_kernel + gemm_bf16_tc_kernel<4 accumulators>", "achieved": round(achieved, 2), "peak": round(peak, 1), "unit": "TFLOP/s",
                         "frac": round(achieved / peak, 4), "peak_source": f"{source} cuBLAS bf16 burst / 6: six bf16 products per f32 product", "traffic": None},
            "reference_published_cpu_gflops": 137.91}


def kernel_attention(ctx, peaks, source, causal=False, steps=20, warmup=5) -> dict:
    """Flash attention forward, B8 H16 S2048 D128 bf16 (config 3)."""
    import torch

    from lighthouse_b200.plan import ArgSpec, Plan
    from lighthouse_b200.workloads import synthetic as I
    from lighthouse_b200.workloads.session import PlanSession

    B, H, S, Dh = 8, 16, 2048, 128
    q, k, v = I.attention_qkv(B, H, H, S, S, Dh, seed=3)
    spec = lambda n: ArgSpec((B, H, S, Dh), "bf16", n)
    plan = Plan("attention_fwd", [spec("o"), spec("q"), spec("k"), spec("v")])
    plan.attention(plan.arg(0), plan.arg(1), plan.arg(2), plan.arg(3), Dh**-0.5, causal)
    sess = PlanSession(plan, ctx=ctx)
    sets = rotating_sets(lambda: [torch.empty(B, H, S, Dh, device="cuda", dtype=torch.bfloat16), q.cuda(), k.cuda(), v.cuda()], 4 * 2 * B * H * S * Dh)
    o = sets[0][0]
    times = time_rotating(ctx, sess, sets, steps, warmup)
    sess.close()
    flops = 4.0 * B * H * S * S * Dh * (0.5 if causal else 1.0)
    mean_s = float(times.mean())
    achieved = flops / mean_s / 1e12
    return {
        "ms": round(mean_s * 1e3, 5), "tflops": round(achieved, 1), "causal": causal, "shape": [B, H, S, Dh],
        "roofline": {"bound": "tensor", "kernel": "attn_fwd_tc3_kernel", "achieved": round(achieved, 1), "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": round(achieved / peaks["bf16_tflops"], 4), "peak_source": f"{source} cuBLAS bf16, burst (kernel timed alone)", "traffic": NCU_TRAFFIC_BYTES["attention_causal" if causal else "attention_full"]},
        "host": (q, k, v, o),
    }


def kernel_rowop(ctx, peaks, source, which: str, M: int, N: int, steps=20, warmup=5) -> dict:
    """Standalone softmax / layer-norm payload (f32, one row kernel): generated as a payload
    module, recognised, run through the native module; HBM roofline with the reference's byte
    model, one read and one write of the matrix (examples/xegpu/softmax.py:24-39)."""
    import torch

    from lighthouse_b200.payload import as_payload_module
    from lighthouse_b200.payload.generators import generate_gpu_layer_norm_payload, generate_gpu_softmax_payload
    from lighthouse_b200.workloads.session import PlanSession

    g = torch.Generator().manual_seed(6)
    x = torch.randn(M, N, generator=g)
    if which == "softmax":
        plan = as_payload_module(generate_gpu_softmax_payload("payload", M, N, "f32")).plans["payload"]
        make = lambda: [torch.empty(M, N, device="cuda"), x.cuda()]
    else:
        plan = as_payload_module(generate_gpu_layer_norm_payload("payload", M, N, "f32")).plans["payload"]
        gamma, beta = torch.randn(N, generator=g).cuda(), torch.randn(N, generator=g).cuda()
        make = lambda: [torch.empty(M, N, device="cuda"), x.cuda(), gamma, beta]
    kinds = [op.kind for op in plan.ops]
    sess = PlanSession(plan, ctx=ctx)
    times = time_rotating(ctx, sess, rotating_sets(make, 2 * 4 * M * N), steps, warmup)
    sess.close()
    mean_s = float(times.mean())
    nbytes = 2.0 * M * N * 4
    achieved = nbytes / mean_s / 1e9
    return {"ms": round(mean_s * 1e3, 5), "gbs": round(achieved, 1), "shape": [M, N], "operators": kinds,
            "roofline": {"bound": "hbm", "kernel": "row_group_kernel", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / peaks["hbm_gbs"], 4), "peak_source": f"{source} copy bandwidth", "traffic": None}}


def kernel_nanogpt(ctx, peaks, source, steps=10, warmup=3) -> dict:
    """nanoGPT forward (config 4: 12 layers, d 768, batch 16, seq 1024, vocab 50304) on one GPU."""
    import torch

    from lighthouse_b200.workloads import decoder as D
    from lighthouse_b200.workloads import synthetic as I
    from lighthouse_b200.workloads.session import PlanSession

    cfg = D.NanoGptConfig()
    w = I.nanogpt_weights(cfg.n_layer, cfg.n_embd, cfg.hidden, cfg.vocab, cfg.block_size, seed=4)
    weights = [t.cuda() for t in D.flatten_nanogpt_args(D.shard_nanogpt_weights(w, cfg))]
    plan = D.build_nanogpt_plan(cfg)
    ids = torch.randint(0, cfg.vocab, (cfg.tokens,), generator=torch.Generator().manual_seed(1)).to(torch.int32).cuda()
    logits = torch.empty(cfg.tokens, cfg.vocab, device="cuda", dtype=torch.float32)
    sess = PlanSession(plan, ctx=ctx)
    sess.set_profiling(True)
    dev_args = [logits, ids] + weights
    torch.cuda.synchronize()  # the context launches on its own stream: operands are complete first
    for _ in range(warmup):
        sess.run(dev_args)
    ctx.sync()
    stream = torch.cuda.ExternalStream(ctx.stream_handle())
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        sess.run(dev_args)
    e1.record(stream)
    ctx.sync()
    ms = e0.elapsed_time(e1) / steps
    roof = gemm_roofline(plan, sess.op_times_ms(), peaks, source)
    sess.close()
    flops = cfg.flops_per_token() * cfg.tokens
    return {"ms": round(ms, 4), "tokens_per_s": round(cfg.tokens / (ms * 1e-3), 1), "model_tflops": round(flops / (ms * 1e-3) / 1e12, 1),
            "algorithmic_tflop_per_step": round(flops / 1e12, 3), "l2": "inputs_exceed_l2 (weights 247 MB, f32 logits 3.3 GB)", "roofline": roof}


def e2e_through_runner(ctx, which: str, repeats: int = 3) -> dict:
    """The reference's own call, timed as a user makes it: ``Runner.execute(name, host numpy
    buffers, callback)`` with ``GPUMemoryManager`` - device allocation, copies from pageable
    host arrays, the payload, the read-back in the callback and the frees, all inside the
    timed region (lighthouse/execution/runner.py:146-224, memory_manager.py:154-168)."""
    import numpy as np

    from lighthouse_b200.execution import GPUMemoryManager, Runner
    from lighthouse_b200.payload.generators import generate_gpu_attention_payload
    from lighthouse_b200.utils.numpy import mlir_to_numpy_dtype
    from lighthouse_b200.workloads.matmul import CudaMatMul

    bf16 = mlir_to_numpy_dtype("bf16")
    rng = np.random.RandomState(8)
    if which == "gemm":
        M = N = K = 4096
        wl = CudaMatMul(M=M, N=N, K=K, ab_type="bf16", c_type="f32", has_bias=True, has_relu=True, accumulate_c=False, truncate_c=True)
        module = wl.payload_module()
        host = [np.zeros((M, N), bf16), (rng.randn(M, K) * 0.02).astype(bf16), (rng.randn(K, N) * 0.02).astype(bf16), rng.randn(N).astype(bf16)]
        flops = 2.0 * M * N * K
    else:
        Z, H, S, Dh = 8, 16, 2048, 128
        module = generate_gpu_attention_payload("payload", Z, H, S, Dh, "bf16")
        host = [np.zeros((Z, H, S, Dh), bf16)] + [rng.randn(Z, H, S, Dh).astype(bf16) for _ in range(3)]
        flops = 4.0 * Z * H * S * S * Dh
    out = np.zeros_like(host[0])
    runner = Runner(module, mem_manager_cls=GPUMemoryManager, context=ctx)
    cb = Runner.get_gpu_argument_access_callback(out)
    runner.execute("payload", host, cb)  # warm-up: module creation, kernel attributes
    t0 = time.perf_counter()
    for _ in range(repeats):
        runner.execute("payload", host, cb)
    dt = (time.perf_counter() - t0) / repeats
    runner.close()
    assert np.isfinite(out.astype(np.float32)).all()
    return {"value": round(flops / dt / 1e12, 3), "unit": "TFLOP/s", "ms_per_call": round(dt * 1e3, 3), "clock": "host wall clock around Runner.execute",
            "h2d_bytes_per_step": int(sum(a.nbytes for a in host)), "d2h_bytes_per_step": int(out.nbytes)}


def kernel_lines(dist: Dist, args) -> dict:
    """Every single-GPU configuration besides the main workload, measured in the same process."""
    from lighthouse_b200.context import CudaContext

    peaks, source = load_peaks()
    ctx = CudaContext(dist.local_rank)
    kernels = {}
    for K in (1024, 2048, 4096, 8192, 16384):  # config 2 and its K sweep
        g = kernel_gemm(ctx, peaks, source, K=K)
        g.pop("host")
        kernels[f"gemm_bias_relu_4096x4096x{K}"] = g
    kernels["gemm_f32_1024x1024x1024"] = kernel_gemm_f32(ctx, peaks, source)
    for causal in (False, True):
        a = kernel_attention(ctx, peaks, source, causal=causal)
        a.pop("host")
        kernels["attention_b8_h16_s2048_d128_" + ("causal" if causal else "full")] = a
    kernels["softmax_f32_32768x4096"] = kernel_rowop(ctx, peaks, source, "softmax", 32768, 4096)
    kernels["layer_norm_f32_16384x768"] = kernel_rowop(ctx, peaks, source, "layer_norm", 16384, 768)
    kernels["layer_norm_f32_131072x768"] = kernel_rowop(ctx, peaks, source, "layer_norm", 131072, 768)
    if args.workload != "nanogpt":
        kernels["nanogpt_forward_config4"] = kernel_nanogpt(ctx, peaks, source)
    kernels["gemm_bias_relu_4096x4096x4096"]["e2e_runner"] = e2e_through_runner(ctx, "gemm")
    kernels["attention_b8_h16_s2048_d128_full"]["e2e_runner"] = e2e_through_runner(ctx, "attention")
    for entry in kernels.values():
        entry.setdefault("l2", L2_NOTE)
    ctx.close()
    return kernels


def run_kernel(args, dist: Dist, which: str) -> dict:
    """N replicas of a single-kernel workload (the path does not shard: no collective)."""
    import torch

    from lighthouse_b200.context import CudaContext

    peaks, source = load_peaks()
    ctx = CudaContext(dist.local_rank)
    sampler = ClockSampler(dist.local_rank)
    sampler.start()
    dist.barrier()
    launches0 = ctx.launch_count
    if which == "gemm":
        r = kernel_gemm(ctx, peaks, source, K=args.k, steps=args.steps, warmup=args.warmup)
        a, b, bias, d = r.pop("host")
        host_ins, dev_out = [a.pin_memory(), b.pin_memory(), bias.pin_memory()], d
        call = lambda ins: ctx.gemm(dev_out, ins[0], ins[1], bias=ins[2], act=1)
        label = workload_description(args)
        metric = "gemm_bias_relu_tflops"
    else:
        r = kernel_attention(ctx, peaks, source, causal=args.causal, steps=args.steps, warmup=args.warmup)
        q, k, v, o = r.pop("host")
        host_ins, dev_out = [q.pin_memory(), k.pin_memory(), v.pin_memory()], o
        call = lambda ins: ctx.attention_fwd(dev_out, ins[0], ins[1], ins[2], 128**-0.5, args.causal)
        label = workload_description(args)
        metric = "attention_fwd_tflops"
    launches = (ctx.launch_count - launches0) * args.steps // (args.steps + args.warmup)
    # end to end through host buffers: H2D of every operand, the kernel, D2H of the result
    stream = torch.cuda.Stream()
    dev_ins = [t.cuda() for t in host_ins]
    host_out = torch.empty(dev_out.shape, dtype=dev_out.dtype).pin_memory()
    with torch.cuda.stream(stream):
        ctx.use_torch_stream()

        def e2e_step():
            for dt, ht in zip(dev_ins, host_ins):
                dt.copy_(ht, non_blocking=True)
            call(dev_ins)
            host_out.copy_(dev_out, non_blocking=True)

        ms_e2e = timed_loop(dist, stream, e2e_step, args.steps, 3)
    clocks = sampler.stop()
    ctx.sync()
    ms = dist.max_over_ranks(r["ms"])
    flops = r["tflops"] * r["ms"] * 1e9  # flops per launch
    n = dist.world
    res = {
        "metric": metric, "value": round(n * flops / (ms * 1e-3) / 1e12, 1), "unit": "TFLOP/s", "n_gpus": n, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": label, "parallelism": "replicas only (independent problems per GPU, no collective)" if n > 1 else "single GPU", "l2": L2_NOTE},
        "roofline": r["roofline"],
        "e2e": {"value": round(n * flops / (ms_e2e / args.steps * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
                "h2d_bytes_per_step": int(n * sum(t.numel() * t.element_size() for t in host_ins)), "d2h_bytes_per_step": int(n * host_out.numel() * host_out.element_size())},
        "gpu_launches": int(launches), "clocks": clocks,
    }
    ctx.close()
    return res


# ------------------------------------------------------------------ CPU baseline (oracle port)
def cpu_sample(which: str, args) -> dict:
    """One bounded sample of the workload on the host cores with the CPU oracle (a port of the
    reference's semantics: its own CPU pipeline needs the MLIR bindings, which are not
    installable here). Returns value in the workload's unit plus what was sampled."""
    import numpy as np
    import torch

    from lighthouse_b200.workloads import synthetic as I
    from oracle import build as oracle_build
    from oracle import inputs as OI
    from oracle import reference_ops as R

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    if which == "gemm":
        rows = 256
        a, b, bias = I.gemm_bf16_normal(rows, 4096, args.k, seed=2)
        A, B, bv = OI.to_np(a), OI.to_np(b), OI.to_np(bias)
        t0 = time.perf_counter()
        oracle_build.matmul_bias_relu(A, B, bv, relu=True)
        dt = time.perf_counter() - t0
        return {"value": 2.0 * rows * 4096 * args.k / dt / 1e12, "unit": "TFLOP/s", "cores": oracle_build.num_threads(), "kind": "port",
                "sample": f"{rows} of 4096 rows of the M=N=4096, K={args.k} problem, C loop nest (i,k,j) with OpenMP over rows, f32"}
    if which == "attention":
        q, k, v = I.attention_qkv(1, 2, 2, 2048, 2048, 128, seed=3)
        t0 = time.perf_counter()
        R.attention(OI.to_np(q), OI.to_np(k), OI.to_np(v), causal=args.causal, io_dtype="bf16")
        dt = time.perf_counter() - t0
        fl = 4.0 * 2 * 2048 * 2048 * 128 * (0.5 if args.causal else 1.0)
        return {"value": fl / dt / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": "2 of the 128 (batch, head) pairs at seq 2048, head_dim 128, numpy f32"}
    if which == "llama":
        from lighthouse_b200.workloads.decoder import LlamaConfig

        cfg = LlamaConfig()
        seq = 512
        w = OI.tree_to_np(I.llama_weights(1, cfg.dim, cfg.n_heads, cfg.n_kv_heads, cfg.ffn, seed=5))
        x = np.random.RandomState(2).randn(1, seq, cfg.dim).astype(np.float32)
        t0 = time.perf_counter()
        R.llama_block(R.round_bf16(x), w["layers"][0], cfg.n_heads, cfg.n_kv_heads, cfg.theta, cfg.eps, "bf16")
        dt = time.perf_counter() - t0
        return {"value": seq / (dt * (args.layers or cfg.n_layer)), "unit": "tokens/s", "cores": cores, "kind": "port",
                "sample": f"1 of {args.layers or cfg.n_layer} layers on batch 1 x seq {seq} (attention is cheaper per token than at seq 4096), numpy/BLAS f32 with bf16 rounding points; tokens/s scaled to the full layer count"}
    from lighthouse_b200.workloads.decoder import NanoGptConfig

    cfg = NanoGptConfig()
    w = OI.tree_to_np(I.nanogpt_weights(2, cfg.n_embd, cfg.hidden, cfg.vocab, cfg.block_size, seed=4))
    ids = np.random.RandomState(1).randint(0, cfg.vocab, size=(1, cfg.seq))
    x = R.embed(ids, w["wte"], w["wpe"])
    ts = []
    for nl in (1, 2):
        t0 = time.perf_counter()
        R.nanogpt_forward(x, w["layers"][:nl], w["gf_g"], w["gf_b"], w["lmw"], w["lmb"], cfg.n_head, cfg.eps, True, "gelu", "bf16", 1)
        ts.append(time.perf_counter() - t0)
    layer = max(ts[1] - ts[0], 1e-6)
    head = max(ts[0] - layer, 0.0)
    nl = args.layers or cfg.n_layer
    return {"value": cfg.seq / (nl * layer + head), "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"batch 1 x seq {cfg.seq}: per-layer time from a 1- and a 2-layer run, lm_head once; tokens/s composed for {nl} layers; numpy/BLAS f32 with bf16 rounding points"}


METRICS = {"llama": "llama_decoder_forward_tokens_per_s", "nanogpt": "nanogpt_decoder_forward_tokens_per_s", "gemm": "gemm_bias_relu_tflops", "attention": "attention_fwd_tflops"}


def workload_description(args, n_gpus: int = 1) -> str:
    """The `config.workload` string of a workload, the same for both arms."""
    from lighthouse_b200.workloads import decoder as D

    if args.workload == "llama":
        cfg = D.LlamaConfig(n_layer=args.layers or 8)
        return "Llama-style decoder stack forward: %d layers, d_model %d, %d q / %d kv heads, head_dim %d, SwiGLU FFN %d, RMSNorm, RoPE, seq %d, batch %d" % (
            cfg.n_layer, cfg.dim, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, cfg.ffn, cfg.seq, cfg.batch)
    if args.workload == "nanogpt":
        cfg = D.NanoGptConfig(n_layer=args.layers or 12)
        return "nanoGPT forward: %d layers, d_model %d, %d heads, GELU MLP x4, pre-LayerNorm, causal, seq %d, batch %d, vocab %d" % (
            cfg.n_layer, cfg.n_embd, cfg.n_head, cfg.seq, cfg.batch, cfg.vocab)
    if args.workload == "gemm":
        return f"bf16 GEMM + bias + ReLU epilogue, M=N=4096, K={args.k}, A,B ~N(0,0.02), bias ~N(0,1), f32 accumulate, bf16 output"
    return f"fused flash-attention forward, bf16, batch 8, heads 16, seq 2048, head_dim 128, {'causal' if args.causal else 'non-causal'}"


def reference_arm(args) -> int:
    """`--impl reference`: the CPU baseline on the host cores, on rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return 0
    for _ in range(min(args.warmup, 1)):
        cpu_sample(args.workload, args)
    t0 = time.perf_counter()
    samples = [cpu_sample(args.workload, args) for _ in range(max(1, min(args.steps, 5)))]
    dt = time.perf_counter() - t0
    value = statistics.mean(s["value"] for s in samples)
    s = samples[0]
    line = {
        "impl": "reference", "metric": METRICS[args.workload], "value": round(value, 6), "unit": s["unit"], "n_gpus": args.gpus, "steps": len(samples),
        "warmup": min(args.warmup, 1), "ms_per_step": round(dt / len(samples) * 1e3, 2), "higher_is_better": True,
        "scaling": "strong" if args.workload in ("llama", "nanogpt") else "weak", "vs_baseline": None, "dtype": "f32 arithmetic on bf16-rounded data", "data": "synthetic",
        "config": {"workload": workload_description(args), "note": "the reference's own CPU pipeline (lh-run through the MLIR ExecutionEngine) is unavailable: mlir-python-bindings cannot be installed offline; this arm times the CPU oracle port of the same path"},
        "cpu_baseline": {"value": round(value, 6), "unit": s["unit"], "cores": s["cores"], "kind": s["kind"], "sample": s["sample"]},
        "e2e": {"value": round(value, 6), "unit": s["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)
    return 0


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=["llama", "nanogpt", "gemm", "attention"], default="llama")
    ap.add_argument("--k", type=int, default=4096, help="K of the GEMM workload (sweep 1024..16384)")
    ap.add_argument("--causal", action="store_true", help="causal mask for the attention workload")
    ap.add_argument("--layers", type=int, default=0, help="override the decoder depth (0 = the configuration's)")
    ap.add_argument("--microbatches", type=int, default=2, help="tensor parallel only: micro-batches whose collectives overlap each other's compute (0: one synchronous all-reduce per contraction)")
    ap.add_argument("--collectives", choices=["fused", "nccl"], default="fused", help="tensor parallel with micro-batches: one multimem kernel per reduce+norm+gather, or NCCL reduce-scatter / all-gather around row kernels")
    ap.add_argument("--timeline", default="", help="decoder workloads: write rank 0's per-operator timeline of the last timed step to this file")
    ap.add_argument("--reserve-sms", type=int, default=8, help="SMs the persistent GEMMs leave to the collectives in the overlapped schedule")
    ap.add_argument("--nanogpt-layout", choices=["dp", "tp"], default="dp", help="nanoGPT on N GPUs: sequences split over the ranks (no collective), or tensor parallel (TP <= 4, 8 GPUs = TP4 x 2 batch halves)")
    ap.add_argument("--no-kernels", action="store_true", help="skip the GEMM / attention kernel lines of the decoder workloads")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="decoder workloads: skip the full-depth check of the result against the CPU oracle")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        return reference_arm(args)

    dist = Dist(args.gpus)
    if args.workload in ("llama", "nanogpt"):
        res = run_decoder(args, dist, args.workload)
    else:
        res = run_kernel(args, dist, args.workload)
    if dist.rank == 0 and dist.world == 1:
        if args.workload in ("llama", "nanogpt") and not args.no_kernels:
            from lighthouse_b200.context import CudaContext

            res["kernels"] = kernel_lines(dist, args)
        if not args.no_cpu_baseline:
            s = cpu_sample(args.workload, args)
            res["cpu_baseline"] = {"value": round(s["value"], 6), "unit": s["unit"], "cores": s["cores"], "kind": s["kind"], "sample": s["sample"]}
    if dist.rank == 0:
        print(json.dumps(res), flush=True)
    dist.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
