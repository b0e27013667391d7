#!/usr/bin/env python
"""Benchmark of the GGML quantized matmul path on B200.

Headline (`value`): weight GB/s of the decode mat-vec sweep — Qwen3-8B-shaped projections
(k=4096 -> n in {4096, 1024, 12288}, k=12288 -> n=4096) x {Q8_0, Q6_K} x m in {1, 2, 4, 8}: 32 mat-vecs per
step, every launch on its own weight buffer (915 MB per step, so each launch finds its weights cold in L2).
One step = one pass over the sweep, replayed from a CUDA graph; timed with CUDA events on the launching stream.

Also reported on the same JSON line: `e2e` (same sweep through the public API with host buffers: activations
written on the host, uploaded, results read back), `roofline` (mat-vec kernel vs measured HBM copy peak),
`cpu_baseline` (the CPU oracle on a bounded sample), `clocks`, `gpu_launches`, and under `extra` the prefill
mat-mat TFLOP/s and the MoE expert-routed tokens/s.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
For N > 1 launch with torch.distributed.run; weights are sharded along N (rows) and every rank's mat-vec kernels
store their columns of the result straight into all ranks' result buffers (peer memory over NVLink, allocated as
torch symmetric memory), with one cross-rank barrier per step ("strong" scaling: the total work is fixed).  If
symmetric memory cannot be set up, every mat-vec output is all-gathered over NCCL instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPES = [(4096, 4096), (1024, 4096), (12288, 4096), (4096, 12288)]  # (n, k)
MS = [1, 2, 4, 8]
TYPE_NAMES = ["Q8_0", "Q6_K"]
BLOCK = {"Q4_0": (32, 18), "Q8_0": (32, 34), "Q6_K": (256, 210)}
METRIC = "q-matvec weight GB/s"


def weight_bytes(t: str, n: int, k: int) -> int:
    qk, bb = BLOCK[t]
    return n * (k // qk) * bb


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx_ = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) >= 9:
                for nm, v in zip(names, r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx_) if mx_ else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def make_weights(t_names, shapes, seed=0):
    """One seeded N(0, 0.02) weight set per (type, shape), packed into GGML blocks on the host."""
    from mlx_native_b200 import ggml_pack as gp

    otype = {"Q4_0": gp.Q4_0, "Q8_0": gp.Q8_0, "Q6_K": gp.Q6_K}
    out = {}
    rng = np.random.default_rng(seed)
    for (n, k) in shapes:
        wf = (rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))
        for t in t_names:
            out[(t, n, k)] = gp.pack(otype[t], wf)
    return out


# --------------------------------------------------------------------------------------------- reference arm
def run_reference(args, rank, world):
    """The CPU oracle (the upstream scalar dequantize + f32 dot path restated in C) on all host threads,
    on a bounded sample of the sweep: every (type, shape) at m = 1, a slice of the weight rows each."""
    if rank != 0:
        return
    from oracle import oracle as orc

    otype = {"Q8_0": orc.Q8_0, "Q6_K": orc.Q6_K}
    cores = os.cpu_count() or 1
    rng = np.random.default_rng(0)
    sample_rows = 512
    items = []
    for t in TYPE_NAMES:
        for (n, k) in SHAPES:
            rows = min(n, sample_rows)
            wf = (rng.standard_normal((rows, k), dtype=np.float32) * np.float32(0.02))
            items.append((t, rows, k, orc.quantize(otype[t], wf, rule="ggml"), rng.standard_normal((1, k)).astype(np.float32)))
    step_bytes = sum(w.size for (_, _, _, w, _) in items)

    def step():
        for (t, rows, k, w, x) in items:
            orc.qmatmul(otype[t], w, x, rows, k, nthreads=cores, want_absdot=False)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    gbs = step_bytes / dt / 1e9
    sample = f"{sample_rows} weight rows of each of the 8 (type, shape) pairs at m=1, {cores} threads"
    line = {"impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "decode mat-vec sweep (Qwen3-8B shapes, Q8_0+Q6_K), CPU scalar oracle, bounded sample"},
            "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# --------------------------------------------------------------------------------------------- our arm
def run_ours(args, rank, world, local_rank):
    import torch

    import mlx_native_b200 as mx
    from mlx_native_b200 import sharding

    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_

        dist = dist_
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    dev = mx.MlxDevice.new(local_rank)
    reg = mx.KernelRegistry.new()
    gt = {"Q8_0": mx.GgmlType.Q8_0, "Q6_K": mx.GgmlType.Q6_K, "Q4_0": mx.GgmlType.Q4_0}

    weights = make_weights(TYPE_NAMES, SHAPES, seed=0)
    rng = np.random.default_rng(1)

    # ---- N > 1: every rank's full-width result buffers live in symmetric memory, so that the other ranks' kernels
    # ---- can store into them (peer stores over NVLink)
    symm = None
    if world > 1 and os.environ.get("MLXN_BENCH_NCCL_GATHER", "0") != "1":
        try:
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer mappings only
            import torch.distributed._symmetric_memory as symm_mem
            total = sum(m * n for (n, k) in SHAPES for m in MS) * len(TYPE_NAMES)
            symm_buf = symm_mem.empty(total, dtype=torch.float32, device=f"cuda:{local_rank}")
            symm_hdl = symm_mem.rendezvous(symm_buf, dist.group.WORLD)
            symm_buf.zero_()
            symm = dict(buf=symm_buf, hdl=symm_hdl, ptrs=[int(p) for p in symm_hdl.buffer_ptrs], off=0)
        except Exception as ex:  # fall back to NCCL all-gathers
            if rank == 0:
                print(f"# symmetric memory unavailable ({ex!r}); using NCCL all-gather per mat-vec", file=sys.stderr)
            symm = None

    # ---- resident data: one weight buffer per launch (sharded by rows across ranks), activations, outputs
    launches = []
    for t in TYPE_NAMES:
        for (n, k) in SHAPES:
            wq = weights[(t, n, k)]
            n_loc = n // world
            w_loc = sharding.shard_weight_bytes(wq, int(gt[t]), n, k, rank, world)
            for m in MS:
                wbuf = dev.alloc_buffer(w_loc.size, mx.DType.U8)
                wbuf.upload(w_loc)
                x = rng.standard_normal((m, k)).astype(np.float32)
                xbuf = dev.alloc_buffer(x.nbytes, mx.DType.F32, [m, k])
                xbuf.upload(x)
                y_loc = y_all = None
                peers = None
                if symm is not None:
                    off = symm["off"]
                    symm["off"] += m * n
                    ybuf = dev.wrap_device_memory(symm["ptrs"][rank] + off * 4, m * n * 4, mx.DType.F32, [m, n])
                    peers = [symm["ptrs"][r] + off * 4 for r in range(world) if r != rank]
                    y_full = symm["buf"][off:off + m * n].view(m, n)
                elif world > 1:
                    y_loc = torch.empty((m, n_loc), dtype=torch.float32, device="cuda")
                    y_all = torch.empty((world * m, n_loc), dtype=torch.float32, device="cuda")
                    ybuf = dev.wrap_device_memory(y_loc.data_ptr(), m * n_loc * 4, mx.DType.F32, [m, n_loc])
                    y_full = None
                else:
                    ybuf = dev.alloc_buffer(m * n_loc * 4, mx.DType.F32, [m, n_loc])
                    y_full = None
                launches.append(dict(t=t, n=n, k=k, m=m, n_loc=n_loc, w=wbuf, x=xbuf, y=ybuf, y_loc=y_loc, y_all=y_all,
                                     peers=peers, y_full=y_full, x_host=x,
                                     params=mx.GgmlQuantizedMatmulParams(m, n_loc, k, gt[t])))
    step_weight_bytes = sum(weight_bytes(L["t"], L["n"], L["k"]) for L in launches)           # whole job
    step_algo_bytes = sum(weight_bytes(L["t"], L["n_loc"], L["k"]) + L["m"] * L["k"] * 4 + L["m"] * L["n_loc"] * 4
                          for L in launches)                                                 # this rank's kernels

    enc = dev.command_encoder()
    ext_stream = torch.cuda.ExternalStream(enc.stream())

    def encode_op(e, L):
        if L["peers"] is not None:
            mx.quantized_matmul_ggml_sharded(e, reg, dev, L["x"], L["w"], L["y"], L["params"], L["n"], rank * L["n_loc"],
                                             L["peers"])
        else:
            mx.quantized_matmul_ggml(e, reg, dev, L["x"], L["w"], L["y"], L["params"])

    def encode_step():
        for L in launches:
            encode_op(enc, L)
            if world > 1 and symm is None:
                with torch.cuda.stream(ext_stream):
                    dist.all_gather_into_tensor(L["y_all"], L["y_loc"])

    graph = None
    if world == 1 or symm is not None:
        encode_step()                      # first touch outside the capture
        enc.commit_and_wait()
        enc.begin_capture()
        encode_step()
        graph = enc.end_capture()

    def rank_barrier_on_stream(stream):
        """All ranks' kernels of the step have finished (their peer stores have landed) before anyone goes on."""
        with torch.cuda.stream(stream):
            symm["hdl"].barrier()

    def run_step():
        if graph is not None:
            graph.launch(enc)
        else:
            encode_step()
        if symm is not None:
            rank_barrier_on_stream(ext_stream)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        run_step()
    enc.commit_and_wait()
    barrier()
    if symm is not None:
        # every rank must hold the same full results: compare with rank 0's copy (tensor-core mat-vecs add split
        # tiles with atomics, so the copies may differ in the last bits, nothing more)
        mine = symm["buf"].clone()
        ref = mine.clone()
        dist.broadcast(ref, src=0)
        scale = float(ref.abs().max().item())
        worst = float((mine - ref).abs().max().item())
        if not (scale > 0 and worst <= 1e-4 * scale):
            raise RuntimeError(f"rank {rank}: assembled results differ from rank 0's: max diff {worst}, scale {scale}")
        # and the columns other ranks stored must be what this rank computes for them: spot-check one launch against
        # an unsharded run of the same mat-vec on this GPU
        L = launches[len(launches) // 2]
        wfull = dev.alloc_buffer(weights[(L["t"], L["n"], L["k"])].size, mx.DType.U8)
        wfull.upload(weights[(L["t"], L["n"], L["k"])])
        ychk = dev.alloc_buffer(L["m"] * L["n"] * 4, mx.DType.F32, [L["m"], L["n"]])
        e2 = dev.command_encoder()
        mx.quantized_matmul_ggml(e2, reg, dev, L["x"], wfull, ychk, mx.GgmlQuantizedMatmulParams(L["m"], L["n"], L["k"], gt[L["t"]]))
        e2.commit_and_wait()
        want = torch.from_numpy(ychk.as_slice(np.float32).reshape(L["m"], L["n"]).copy()).cuda()
        diff = float((L["y_full"] - want).abs().max().item())
        if not diff <= 1e-4 * float(want.abs().max().item()):
            raise RuntimeError(f"rank {rank}: sharded result differs from the unsharded mat-vec: {diff}")
        del wfull, ychk

    del weights
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    mx.reset_counters()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(ext_stream):
        ev0.record()
    for _ in range(args.steps):
        run_step()
    with torch.cuda.stream(ext_stream):
        ev1.record()
    enc.commit_and_wait()
    barrier()
    ms_total = ev0.elapsed_time(ev1)
    n_launch = mx.kernel_launch_count()
    clocks = sampler.stop() if rank == 0 else None
    if dist is not None:
        tt = torch.tensor([ms_total], device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms_total = float(tt.item())
    ms_step = ms_total / args.steps
    value = step_weight_bytes / (ms_step * 1e-3) / 1e9

    # ---- e2e: the same sweep through the public API with host buffers, copies inside the timed region
    e2e_steps = max(3, min(args.steps, 20))
    h2d = sum(L["m"] * L["k"] * 4 for L in launches)
    d2h = sum(L["m"] * (L["n"] if symm is not None else L["n_loc"]) * 4 for L in launches)

    # The public API's own graph capture records the uploads of the (host-written) activations as part of the
    # graph, and a committed command buffer brings results with a host view back: one step is "write the
    # activations on the host, replay, wait, read the results on the host".
    e2e_enc = dev.command_encoder()
    e2e_stream = torch.cuda.ExternalStream(e2e_enc.stream())

    def write_inputs():
        for L in launches:
            L["x"].as_mut_slice(np.float32)[:] = L["x_host"].reshape(-1)      # host write -> upload at bind / replay

    def e2e_encode():
        for L in launches:
            encode_op(e2e_enc, L)
            if world > 1 and symm is None:
                with torch.cuda.stream(e2e_stream):
                    dist.all_gather_into_tensor(L["y_all"], L["y_loc"])

    e2e_graph = None
    if world == 1 or symm is not None:
        for L in launches:                                                    # create the pinned shadows up front
            L["y"].as_slice(np.float32)
        write_inputs()
        e2e_encode()
        e2e_enc.commit_and_wait()
        write_inputs()
        e2e_enc.begin_capture()
        e2e_encode()
        e2e_graph = e2e_enc.end_capture()

    def e2e_step():
        write_inputs()
        if e2e_graph is not None:
            e2e_graph.launch(e2e_enc)
        else:
            e2e_encode()
        if symm is not None:
            rank_barrier_on_stream(e2e_stream)
        e2e_enc.commit_and_wait()
        acc = 0.0
        for L in launches:
            if world > 1 and symm is None:
                acc += float(L["y_all"][0, 0].item())                      # device -> host read of the result
            else:
                acc += float(L["y"].as_slice(np.float32)[0])               # host view, fetched back by the commit
        return acc

    for _ in range(2):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    if dist is not None:
        tt = torch.tensor([e2e_s], device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_s = float(tt.item())
    e2e_value = step_weight_bytes / e2e_s / 1e9

    sharded = None
    if world > 1 and not args.no_extra:
        try:
            sharded = sharded_extra(mx, dev, reg, torch, dist, rank, world, enc, ext_stream)
        except Exception as ex:  # the headline stands on its own
            sharded = {"error": repr(ex)}
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    hbm_peak, tf_peak, peak_kind = measured_peaks()
    achieved = step_algo_bytes / (ms_step * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "decode mat-vec sweep: Qwen3-8B projections (4096->4096, 4096->1024, 4096->12288, "
                               "12288->4096) x {Q8_0,Q6_K} x m in {1,2,4,8}; 32 mat-vecs per step",
                   "weight_bytes_per_step": step_weight_bytes, "l2": "each launch has its own weight buffer: 915 MB of "
                   "distinct weights per step, larger than L2", "launch": "CUDA graph replay" if graph is not None else
                   "direct launches + NCCL all-gather per mat-vec",
                   "exchange": "none" if world == 1 else ("peer stores from the mat-vec kernels into every rank's result "
                   "buffer (symmetric memory) + one cross-rank barrier per step" if symm is not None else
                   "NCCL all-gather per mat-vec"), "parallelism": f"n-shard x{world}"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                     "traffic": step_algo_bytes * 1.01, "traffic_note": "ncu dram__bytes_read+write of qmv_tc_kernel is 1.008x (Q8_0) "
                     "and 1.011x (Q6_K) its algorithmic bytes (profiles/qmv_tc_*_full.md); scaled to the step", "peak_kind": f"{peak_kind} copy bandwidth", "kernel": "qmv_tc_kernel (+ qmv_tc_pack_kernel)",
                     "note": "achieved = (weight + activation + output bytes of the 32 launches) / event-timed step"},
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_s * 1e3},
        "gpu_launches": int(n_launch),
        "clocks": clocks,
    }

    if world == 1:
        line["cpu_baseline"] = cpu_baseline()
        if not args.no_extra:
            try:
                line["extra"] = extra_numbers(mx, dev, reg, torch, tf_peak, hbm_peak)
            except Exception as ex:  # the headline stands on its own
                line["extra"] = {"error": repr(ex)}
    if sharded is not None:
        line["extra"] = sharded
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def sharded_extra(mx, dev, reg, torch, dist, rank, world, enc, ext_stream):
    """Secondary multi-GPU figures, every rank taking part:
    the expert-sharded MoE FFN layer (128 experts / world per rank, local routing filter, one all-reduce of the
    [T, hidden] partial sums as the combine) and the N-sharded Q6_K lm_head mat-vec (151936 x 5120, m = 1, peer
    stores into every rank's logits + one cross-rank barrier)."""
    from mlx_native_b200 import sharding
    from mlx_native_b200.profile_case import random_blocks

    out = {}
    rng = np.random.default_rng(11)          # same seed on every rank: replicated activations and logits

    def timed(step, reps=10, warm=3):
        for _ in range(warm):
            step()
        enc.commit_and_wait()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(ext_stream):
            e0.record()
        for _ in range(reps):
            step()
        with torch.cuda.stream(ext_stream):
            e1.record()
        enc.commit_and_wait()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / reps * 1e-3], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- expert-sharded MoE FFN layer
    E, top_k, hidden, ffn = 128, 8, 2048, 768
    lo, cnt = sharding.shard_experts(E, rank, world)
    wrng = np.random.default_rng(100 + rank)
    w = {}
    for name, t, rows, cols in (("gate", "Q4_0", cnt * ffn, hidden), ("up", "Q4_0", cnt * ffn, hidden), ("down", "Q6_K", cnt * hidden, ffn)):
        blk = random_blocks(wrng, t, rows, cols)
        w[name] = dev.alloc_buffer(blk.size, mx.DType.U8)
        w[name].upload(blk)
        w[name + "_stride"] = blk.size // cnt
    moe = {}
    for T in (512, 1):
        logits = rng.standard_normal((T, E)).astype(np.float32)
        lg = dev.alloc_buffer(logits.nbytes, mx.DType.F32)
        lg.upload(logits)
        x = rng.standard_normal((T, hidden)).astype(np.float32)
        xb = dev.alloc_buffer(x.nbytes, mx.DType.F32)
        xb.upload(x)
        pairs = T * top_k
        ids = dev.alloc_buffer(pairs * 4, mx.DType.U32)
        lids = dev.alloc_buffer(pairs * 4, mx.DType.U32)
        rw = dev.alloc_buffer(pairs * 4, mx.DType.F32)
        yg = dev.alloc_buffer(pairs * ffn * 4, mx.DType.F32)
        yu = dev.alloc_buffer(pairs * ffn * 4, mx.DType.F32)
        act = dev.alloc_buffer(pairs * ffn * 4, mx.DType.F32)
        yd = dev.alloc_buffer(pairs * hidden * 4, mx.DType.F32)
        out_t = torch.zeros((T, hidden), dtype=torch.float32, device="cuda")
        outb = dev.wrap_device_memory(out_t.data_ptr(), T * hidden * 4, mx.DType.F32, [T, hidden])
        pg = mx.GgmlQuantizedMatmulIdParams(T, top_k, ffn, hidden, cnt, w["gate_stride"], mx.GgmlType.Q4_0)
        pd = mx.GgmlQuantizedMatmulIdParams(pairs, 1, hidden, ffn, cnt, w["down_stride"], mx.GgmlType.Q6_K)

        def layer(e):
            mx.moe_softmax_topk(e, reg, dev, lg, ids, rw, T, E, top_k)            # replicated routing
            mx.moe_expert_shard_route(e, reg, dev, ids, lids, pairs, lo, cnt)     # dispatch = local filter
            mx.quantized_matmul_id_ggml(e, reg, dev, xb, w["gate"], lids, yg, pg)
            mx.quantized_matmul_id_ggml(e, reg, dev, xb, w["up"], lids, yu, pg)
            mx.silu_mul(e, reg, dev, yg, yu, act, pairs * ffn)
            mx.quantized_matmul_id_ggml(e, reg, dev, act, w["down"], lids, yd, pd)
            mx.moe_weighted_reduce_local(e, reg, dev, rw, yd, lids, outb, T, top_k, hidden)

        layer(enc)
        enc.commit_and_wait()
        enc.begin_capture()
        layer(enc)
        g = enc.end_capture()

        def step():
            g.launch(enc)
            with torch.cuda.stream(ext_stream):
                dist.all_reduce(out_t)                                             # combine

        sec = timed(step)
        if not bool(torch.isfinite(out_t).all().item()):
            raise RuntimeError("expert-sharded MoE layer produced non-finite values")
        moe[f"m{T}"] = {"tokens_per_s": T / sec, "ms_per_layer": sec * 1e3, "experts_per_rank": cnt,
                        "combine": "NCCL all-reduce of the [T, hidden] partial sums"}
    out["moe_ffn_layer_expert_sharded"] = moe

    # ---- N-sharded lm_head, Q6_K 151936 x 5120, m = 1
    n, k, m = 151936, 5120, 1
    try:
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        n_loc = n // world
        blk = random_blocks(wrng, "Q6_K", n_loc, k)
        wb = dev.alloc_buffer(blk.size, mx.DType.U8)
        wb.upload(blk)
        x = rng.standard_normal((m, k)).astype(np.float32)
        xb = dev.alloc_buffer(x.nbytes, mx.DType.F32, [m, k])
        xb.upload(x)
        buf = symm_mem.empty(m * n, dtype=torch.float32, device=f"cuda:{torch.cuda.current_device()}")
        hdl = symm_mem.rendezvous(buf, dist.group.WORLD)
        buf.zero_()
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        yb = dev.wrap_device_memory(ptrs[rank], m * n * 4, mx.DType.F32, [m, n])
        peers = [ptrs[r] for r in range(world) if r != rank]
        prm = mx.GgmlQuantizedMatmulParams(m, n_loc, k, mx.GgmlType.Q6_K)

        def step():
            mx.quantized_matmul_ggml_sharded(enc, reg, dev, xb, wb, yb, prm, n, rank * n_loc, peers)
            with torch.cuda.stream(ext_stream):
                hdl.barrier()

        sec = timed(step)
        nz = int((buf != 0).sum().item())
        out["lm_head_q6k_m1_n_sharded"] = {"us": sec * 1e6, "weight_GBps_all_ranks": n * (k // 256) * 210 / sec / 1e9,
                                           "logits_filled": nz, "of": m * n,
                                           "exchange": "peer stores from the mat-vec kernel + one barrier"}
    except Exception as ex:
        out["lm_head_q6k_m1_n_sharded"] = {"error": repr(ex)}
    return out


def cpu_baseline():
    from oracle import oracle as orc

    cores = os.cpu_count() or 1
    rng = np.random.default_rng(0)
    n, k = 2048, 4096
    wf = (rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))
    x = rng.standard_normal((1, k)).astype(np.float32)
    total_b, total_t = 0, 0.0
    for t, ot in (("Q8_0", orc.Q8_0), ("Q6_K", orc.Q6_K)):
        w = orc.quantize(ot, wf, rule="ggml")
        orc.qmatmul(ot, w, x, n, k, nthreads=cores, want_absdot=False)
        reps = 5
        t0 = time.perf_counter()
        for _ in range(reps):
            orc.qmatmul(ot, w, x, n, k, nthreads=cores, want_absdot=False)
        total_t += time.perf_counter() - t0
        total_b += reps * w.size
    return {"value": total_b / total_t / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": f"2048x4096 Q8_0 and Q6_K weights, m=1, 5 repetitions each, {cores} host threads"}


def extra_numbers(mx, dev, reg, torch, tf_peak, hbm_peak):
    """Secondary figures: prefill mat-mat TFLOP/s (Q4_0 and Q6_K, m=512 and 2048, 4096x4096) and
    MoE expert-routed tokens/s (128 experts, top-8, hidden 2048, ffn 768, m=512 and m=1)."""
    from mlx_native_b200 import ggml_pack as gp

    out = {}
    rng = np.random.default_rng(3)
    otype = {"Q4_0": gp.Q4_0, "Q6_K": gp.Q6_K}
    gt = {"Q4_0": mx.GgmlType.Q4_0, "Q6_K": mx.GgmlType.Q6_K}

    def timed(fn, reps=10, warm=3, inner=4):
        """Median device time of one call of `fn`: `inner` calls are captured into one CUDA graph, so that the graph
        launch and the first call's start-up latency are shared (as in a real sequence of calls)."""
        e = dev.command_encoder()
        for _ in range(warm):
            fn(e)
        e.commit_and_wait()
        e.begin_capture()
        for _ in range(inner):
            fn(e)
        g = e.end_capture()
        g.launch(e)
        e.commit_and_wait()
        ts = []
        for _ in range(reps):
            g.launch(e)
            ts.append(e.commit_wait_with_gpu_time() / inner)
        return statistics.median(ts)

    mm = {}
    for (n, k, ms) in ((4096, 4096, (512, 2048)), (12288, 4096, (2048,)), (4096, 12288, (2048,))):
        wf = (rng.standard_normal((512, k), dtype=np.float32) * np.float32(0.02))
        for t in ("Q4_0", "Q6_K"):
            wq = np.tile(gp.pack(otype[t], wf), n // 512)   # timing does not depend on the values
            wb = dev.alloc_buffer(wq.size, mx.DType.U8)
            wb.upload(wq)
            for m in ms:
                x = rng.standard_normal((m, k)).astype(np.float32)
                xb = dev.alloc_buffer(x.nbytes, mx.DType.F32)
                xb.upload(x)
                yb = dev.alloc_buffer(m * n * 4, mx.DType.F32)
                p = mx.GgmlQuantizedMatmulParams(m, n, k, gt[t])
                sec = timed(lambda e: mx.quantized_matmul_ggml(e, reg, dev, xb, wb, yb, p))
                tf = 2.0 * m * n * k / sec / 1e12
                mm[f"{t}_m{m}_n{n}_k{k}"] = {"tflops": tf, "ms": sec * 1e3, "frac_of_measured_bf16_peak": tf / tf_peak}
            del wb
    out["qmm"] = mm

    # MoE FFN: gate + up (Q4_0 [768 x 2048] per expert), down (Q6_K [2048 x 768] per expert)
    E, top_k, hidden, ffn = 128, 8, 2048, 768
    w1 = gp.pack(gp.Q4_0, (rng.standard_normal((ffn, hidden), dtype=np.float32) * np.float32(0.02)))
    w2 = gp.pack(gp.Q6_K, (rng.standard_normal((hidden, ffn), dtype=np.float32) * np.float32(0.02)))
    wg = dev.alloc_buffer(w1.size * E, mx.DType.U8)
    wu = dev.alloc_buffer(w1.size * E, mx.DType.U8)
    wd = dev.alloc_buffer(w2.size * E, mx.DType.U8)
    for e_ in range(E):  # the same expert bytes repeated: timing does not depend on the values
        wg.upload(w1, e_ * w1.size)
        wu.upload(w1, e_ * w1.size)
        wd.upload(w2, e_ * w2.size)
    moe = {}
    for T in (1, 512):
        logits = rng.standard_normal((T, E)).astype(np.float32)
        lg = dev.alloc_buffer(logits.nbytes, mx.DType.F32)
        lg.upload(logits)
        x = rng.standard_normal((T, hidden)).astype(np.float32)
        xb = dev.alloc_buffer(x.nbytes, mx.DType.F32)
        xb.upload(x)
        ids = dev.alloc_buffer(T * top_k * 4, mx.DType.U32)
        rw = dev.alloc_buffer(T * top_k * 4, mx.DType.F32)
        yg = dev.alloc_buffer(T * top_k * ffn * 4, mx.DType.F32)
        yu = dev.alloc_buffer(T * top_k * ffn * 4, mx.DType.F32)
        act = dev.alloc_buffer(T * top_k * ffn * 4, mx.DType.F32)
        yd = dev.alloc_buffer(T * top_k * hidden * 4, mx.DType.F32)
        outb = dev.alloc_buffer(T * hidden * 4, mx.DType.F32)
        pg = mx.GgmlQuantizedMatmulIdParams(T, top_k, ffn, hidden, E, w1.size, mx.GgmlType.Q4_0)
        pd = mx.GgmlQuantizedMatmulIdParams(T * top_k, 1, hidden, ffn, E, w2.size, mx.GgmlType.Q6_K)

        def layer(e):
            mx.moe_softmax_topk(e, reg, dev, lg, ids, rw, T, E, top_k)
            mx.quantized_matmul_id_ggml(e, reg, dev, xb, wg, ids, yg, pg)
            mx.quantized_matmul_id_ggml(e, reg, dev, xb, wu, ids, yu, pg)
            mx.silu_mul(e, reg, dev, yg, yu, act, T * top_k * ffn)
            mx.quantized_matmul_id_ggml(e, reg, dev, act, wd, ids, yd, pd)
            mx.moe_weighted_reduce(e, reg, dev, rw, yd, outb, T, top_k, hidden)

        sec = timed(layer)
        active = min(E, T * top_k)
        wbytes = active * (2 * w1.size + w2.size) if T == 1 else E * (2 * w1.size + w2.size)
        moe[f"m{T}"] = {"tokens_per_s": T / sec, "ms_per_layer": sec * 1e3, "expert_weight_GBps": wbytes / sec / 1e9,
                        "frac_of_measured_hbm_peak": wbytes / sec / 1e9 / hbm_peak}
    out["moe_ffn_layer"] = moe

    # lm_head: Q6_K 151936 x 5120 (638 MB), m = 1 (mat-vec, HBM-bound) and m = 256 (mat-mat)
    from mlx_native_b200.profile_case import random_blocks
    n, k = 151936, 5120
    blk = random_blocks(rng, "Q6_K", n, k)
    wb = dev.alloc_buffer(blk.size, mx.DType.U8)
    wb.upload(blk)
    lm = {}
    for m in (1, 256):
        x = rng.standard_normal((m, k)).astype(np.float32)
        xb = dev.alloc_buffer(x.nbytes, mx.DType.F32)
        xb.upload(x)
        yb = dev.alloc_buffer(m * n * 4, mx.DType.F32)
        p = mx.GgmlQuantizedMatmulParams(m, n, k, mx.GgmlType.Q6_K)
        sec = timed(lambda e: mx.quantized_matmul_ggml(e, reg, dev, xb, wb, yb, p), inner=2)
        lm[f"m{m}"] = {"us": sec * 1e6, "weight_GBps": blk.size / sec / 1e9, "frac_of_measured_hbm_peak": blk.size / sec / 1e9 / hbm_peak,
                       "tflops": 2.0 * m * n * k / sec / 1e12}
    out["lm_head_q6k"] = lm
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip the secondary mat-mat / MoE figures")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
