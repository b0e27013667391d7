#!/usr/bin/env python
"""Benchmark of the GGML quantized matmul path on B200.

Headline (`value`): weight GB/s of the decode mat-vec sweep — Qwen3-8B-shaped projections
(k=4096 -> n in {4096, 1024, 12288}, k=12288 -> n=4096) x {Q8_0, Q6_K} x m in {1, 2, 4, 8}: 32 mat-vecs per
step, every launch on its own weight buffer (915 MB per step, so each launch finds its weights cold in L2).
One step = one pass over the sweep, replayed from a CUDA graph; timed with CUDA events on the launching stream.

The 32 mat-vecs of a step are independent, so the encoder may overlap them, and mat-vecs of one block type and
activation-row class that follow one another leave as one kernel; the sweep is therefore encoded row count by row
count.  The same sweep is also timed as a DEPENDENT CHAIN (all 32 write one shared result buffer, so each waits for
the one ahead, as the projections of a decoder layer do): that figure is the one in `roofline`; the independent one
is `value` and `roofline_independent`.

Also reported on the same JSON line: `e2e` (same sweep through the public API with host buffers: activations
written on the host, uploaded, results read back; on one GPU four steps are in flight, commit / wait_until_completed
on four encoders, so one step's copy back and host read overlap the next step's upload and kernels), `cpu_baseline` (the CPU oracle on a bounded sample, all host
threads and one thread), `clocks`, `gpu_launches`, and `roofline_by_config`: one entry per benchmark configuration
(Q4_0 4096x4096 mat-vec; the sweep; the twelve prefill mat-mat cells in TFLOP/s against the measured bf16 burst and the
nominal 2250; the MoE FFN layer in tokens/s and expert-weight GB/s; the lm_head at m = 1 and m = 256).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
  python bench.py --case mv|mm|moe|moe_layer|cmp [args]     small fixed workloads for profiler captures (see run_case)
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
BLOCK = {"Q4_0": (32, 18), "Q8_0": (32, 34), "Q6_K": (256, 210), "Q4_K": (256, 144)}
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


def traffic_ratio(launches):
    """DRAM bytes per algorithmic byte of the mat-vec kernels, from the ncu captures summarised in
    profiles/matvec_dram_traffic.md (rows `| kernel | type | shape | m | algorithmic MB | dram MB | ratio |`),
    weighted by the sweep's bytes per block type."""
    table = {}
    try:
        with open(os.path.join(ROOT, "profiles", "matvec_dram_traffic.md")) as f:
            for line in f:
                cells = [c.strip() for c in line.strip().strip("|").split("|")]
                if len(cells) >= 7 and cells[0].startswith("qmv_"):
                    table.setdefault(cells[1], []).append(float(cells[6]))
    except Exception:
        return None, "profiles/matvec_dram_traffic.md not found"
    tot = num = 0.0
    for L in launches:
        b = weight_bytes(L["t"], L["n_loc"], L["k"])
        rs = table.get(L["t"])
        if rs:
            tot += b
            num += b * (sum(rs) / len(rs))
    if tot == 0:
        return None, "no capture for these block types in profiles/matvec_dram_traffic.md"
    return num / tot, ("dram__bytes_read+write per algorithmic byte from profiles/matvec_dram_traffic.md (mean per block "
                       "type over the captured shapes), scaled to the step")


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
    cores = os.cpu_count() or 1
    items, step_bytes, sample_rows = reference_sample()
    dt = time_oracle(items, cores, steps=args.steps, warmup=args.warmup)
    gbs = step_bytes / dt / 1e9
    sample = (f"the whole sweep cut to {sample_rows} weight rows per mat-vec ({step_bytes / 1e6:.1f} MB of weights per pass), "
              f"{cores} threads")
    line = {"impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": sweep_config(args.gpus),
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
        import datetime
        # (a lost rank ends the others' next collective with an error after three minutes instead of the default ten)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=datetime.timedelta(seconds=180))
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
    # encoded row count by row count, type by type: neighbours in the sweep can then leave as one kernel
    for (m, t) in [(m, t) for m in MS for t in TYPE_NAMES]:
        for (n, k) in SHAPES:
            wq = weights[(t, n, k)]
            n_loc = n // world
            w_loc = sharding.shard_weight_bytes(wq, int(gt[t]), n, k, rank, world)
            for _once in (0,):
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
                enc.memory_barrier()          # the mat-vec may sit on the encoder's other lane (or still be pending)
                with torch.cuda.stream(ext_stream):
                    dist.all_gather_into_tensor(L["y_all"], L["y_loc"])

    graph = None
    if world == 1 or symm is not None:
        encode_step()                      # first touch outside the capture
        enc.commit_and_wait()
        enc.begin_capture()
        encode_step()
        graph = enc.end_capture()

    pbar = sharding.PeerBarrier(local_rank) if symm is not None else None

    def rank_barrier_on_stream(stream, e=None):
        """All ranks' kernels of the step have finished (their peer stores have landed) before anyone goes on: the
        library's own barrier kernel over a flag array in symmetric memory (bounded wait, plain peer stores)."""
        pbar.wait(e if e is not None else enc)

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

    if world > 1:
        # every rank's assembled results against the CPU oracle, on rows around every shard boundary and the last rows
        from oracle import oracle as orc
        otype = {"Q8_0": orc.Q8_0, "Q6_K": orc.Q6_K}
        for L in launches[::5]:
            t, n, k, m, n_loc = L["t"], L["n"], L["k"], L["m"], L["n_loc"]
            rows = sorted({r for b in range(world) for r in (b * n_loc, b * n_loc + 1, (b + 1) * n_loc - 1)} | {n - 1})
            rb = weight_bytes(t, 1, k)
            wq = weights[(t, n, k)]
            wsel = np.concatenate([wq[r * rb:(r + 1) * rb] for r in rows])
            ref, ad = orc.qmatmul(otype[t], wsel, L["x_host"], len(rows), k, nthreads=4)
            if L["y_full"] is not None:
                got = L["y_full"].cpu().numpy()[:, rows]
            else:   # NCCL fallback: [world * m, n_loc] gathered blocks
                ya = L["y_all"].cpu().numpy().reshape(world, m, n_loc)
                got = np.stack([ya[r // n_loc, :, r % n_loc] for r in rows], axis=1)
            err = float(np.max(np.abs(got.astype(np.float64) - ref) / np.maximum(ad, 1e-30)))
            if not err <= 1e-5:
                raise RuntimeError(f"rank {rank}: sharded {t} {n}x{k} m={m} differs from the oracle: normalised error {err:.3e}")
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

    # ---- the same sweep as a dependent chain: every mat-vec writes the one shared result buffer, so each waits for
    # ---- the one ahead (write-after-write), as the projections of a decoder layer wait for one another
    ms_chain = None
    chain_launches = None
    if world == 1:
        shared = dev.alloc_buffer(max(L["m"] * L["n_loc"] for L in launches) * 4, mx.DType.F32)

        def encode_chain():
            for L in launches:
                yv = shared.slice_view(0, L["m"] * L["n_loc"])
                mx.quantized_matmul_ggml(enc, reg, dev, L["x"], L["w"], yv, L["params"])

        encode_chain()
        enc.commit_and_wait()
        enc.begin_capture()
        encode_chain()
        cgraph = enc.end_capture()
        for _ in range(3):
            cgraph.launch(enc)
        enc.commit_and_wait()
        mx.reset_counters()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(ext_stream):
            c0.record()
        for _ in range(args.steps):
            cgraph.launch(enc)
        with torch.cuda.stream(ext_stream):
            c1.record()
        enc.commit_and_wait()
        ms_chain = c0.elapsed_time(c1) / args.steps
        chain_launches = mx.kernel_launch_count()

    # ---- e2e: the same sweep through the public API with host buffers, copies inside the timed region
    e2e_steps = max(8, min(args.steps, 100))
    h2d = sum(L["m"] * L["k"] * 4 for L in launches)
    d2h = sum(L["m"] * (L["n"] if symm is not None else L["n_loc"]) * 4 for L in launches)

    # The public API's own graph capture records the uploads of the (host-written) activations as part of the
    # graph, and a committed command buffer brings results with a host view back: one step is "write the
    # activations on the host, replay, wait, read the results on the host".
    e2e_enc = dev.command_encoder()
    e2e_stream = torch.cuda.ExternalStream(e2e_enc.stream())
    e2e_in_flight = 1
    if world == 1 or symm is not None:
        # Four steps in flight (upstream's commit / wait_until_completed pair, src/encoder.rs:2022-2050): four command
        # encoders, each with one arena for the step's activations and one for its results, the mat-vecs working on
        # views of them (MlxBuffer::slice_view, src/buffer.rs:187-197).  Step i is: wait for step i - 4 and read its
        # results on the host; write the activations on the host (all 2.9 MB), replay the encoder's graph (one upload,
        # 32 mat-vecs), commit (one copy back).  Every step uploads its own inputs and reads its own results; measured
        # per step on one GPU: 0.66 ms with one step in flight, 0.43 / 0.35 / 0.32 ms with two / three / four (the kernels
        # alone take 0.33 ms).
        # On N GPUs every set's result arena is a symmetric-memory buffer of its own (the other ranks' kernels store their
        # columns into it) with its own cross-rank barrier flags, and a step is bracketed by two barriers: one in front
        # of the kernels (every rank has finished copying the set's previous results back, so they may be overwritten)
        # and one behind them (every rank's columns have arrived, so the copy back may start).
        e2e_in_flight = 4
        x_host = np.concatenate([L["x_host"].reshape(-1) for L in launches])
        n_res = sum(L["m"] * (L["n"] if symm is not None else L["n_loc"]) for L in launches)      # floats per result arena
        sets = []
        for s_i in range(e2e_in_flight):
            xa = dev.alloc_buffer(h2d, mx.DType.F32)
            if symm is not None:
                import torch.distributed._symmetric_memory as symm_mem
                sbuf = symm_mem.empty(n_res, dtype=torch.float32, device=f"cuda:{local_rank}")
                shdl = symm_mem.rendezvous(sbuf, dist.group.WORLD)
                sbuf.zero_()
                sptrs = [int(p_) for p_ in shdl.buffer_ptrs]
                ya = dev.wrap_device_memory(sptrs[rank], n_res * 4, mx.DType.F32)
                set_bar = sharding.PeerBarrier(local_rank)
            else:
                sbuf = shdl = sptrs = set_bar = None
                ya = dev.alloc_buffer(d2h, mx.DType.F32)
            ops, y_offs, xo, yo = [], [], 0, 0
            for L in launches:
                width = L["n"] if symm is not None else L["n_loc"]
                peers_s = [sptrs[r] + yo * 4 for r in range(world) if r != rank] if symm is not None else None
                ops.append(dict(L, x=xa.slice_view(xo * 4, L["m"] * L["k"]), y=ya.slice_view(yo * 4, L["m"] * width), peers=peers_s))
                y_offs.append(yo)
                xo += L["m"] * L["k"]
                yo += L["m"] * width
            e = dev.command_encoder()
            ya.as_slice(np.float32)                                           # create the pinned shadow up front
            xa.as_mut_slice(np.float32)[:] = x_host
            for op in ops:                                                    # first touch outside the capture
                encode_op(e, op)
            e.commit_and_wait()
            xa.as_mut_slice(np.float32)[:] = x_host
            e.begin_capture()
            for op in ops:
                encode_op(e, op)
            sets.append(dict(x=xa, y=ya, enc=e, graph=e.end_capture(), y_offs=y_offs, bar=set_bar, keep=(sbuf, shdl)))
        barrier()

        def submit(st):
            st["x"].as_mut_slice(np.float32)[:] = x_host                      # host write -> upload at replay
            if st["bar"] is not None:
                st["bar"].wait(st["enc"])                                     # the set's previous results are read everywhere
            st["graph"].launch(st["enc"])
            if st["bar"] is not None:
                st["bar"].wait(st["enc"])                                     # every rank's columns have arrived
            st["enc"].commit()                                                # results with a host view are copied back

        def collect(st):
            st["enc"].wait_until_completed()
            res = st["y"].as_slice(np.float32)                                # host view, fetched back by the commit
            return float(sum(res[o] for o in st["y_offs"]))

        def e2e_run(n):
            acc = 0.0
            D = e2e_in_flight
            for i in range(n):
                if i >= D:
                    acc += collect(sets[(i - D) % D])                         # the set's previous step, before its reuse
                submit(sets[i % D])
            for i in range(max(0, n - D), n):
                acc += collect(sets[i % D])
            return acc

        e2e_run(2 * e2e_in_flight)
        barrier()
        t0 = time.perf_counter()
        e2e_run(e2e_steps)
        barrier()
        e2e_s = (time.perf_counter() - t0) / e2e_steps
        if dist is not None:
            tt = torch.tensor([e2e_s], device="cuda")
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            e2e_s = float(tt.item())
        # what came back to the host is what the device-timed sweep left in its own result buffers (same inputs)
        for st in sets:
            res = st["y"].as_slice(np.float32)
            for L, o in zip(launches, st["y_offs"]):
                want = (L["y_full"].cpu().numpy() if symm is not None else L["y"].download(np.float32)).reshape(-1)
                got = res[o:o + want.size]
                scale = max(float(np.max(np.abs(want))), 1e-30)
                if not np.all(np.isfinite(got)) or float(np.max(np.abs(got - want))) > 1e-5 * scale:
                    raise RuntimeError(f"rank {rank}: e2e result of {L['t']} {L['n']}x{L['k']} m={L['m']} differs from the "
                                       f"device-timed sweep's: {float(np.max(np.abs(got - want))) / scale:.3e} of its scale")
    else:
        # (no symmetric memory: direct launches and one NCCL all-gather per mat-vec, one step at a time)
        def e2e_step():
            for L in launches:
                L["x"].as_mut_slice(np.float32)[:] = L["x_host"].reshape(-1)      # host write -> upload at bind
            for L in launches:
                encode_op(e2e_enc, L)
                e2e_enc.memory_barrier()
                with torch.cuda.stream(e2e_stream):
                    dist.all_gather_into_tensor(L["y_all"], L["y_loc"])
            e2e_enc.commit_and_wait()
            return sum(float(L["y_all"][0, 0].item()) for L in launches)       # device -> host read of the results

        for _ in range(2):
            e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        barrier()
        e2e_s = (time.perf_counter() - t0) / e2e_steps
        tt = torch.tensor([e2e_s], device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_s = float(tt.item())
    e2e_value = step_weight_bytes / e2e_s / 1e9

    sharded = None
    if world > 1 and not args.no_extra:
        try:
            sharded = sharded_extra(mx, dev, reg, torch, dist, rank, world, enc, ext_stream, pbar)
        except Exception as ex:  # the headline stands on its own
            sharded = {"error": repr(ex)}
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    hbm_peak, tf_peak, peak_kind = measured_peaks()
    ratio, ratio_note = traffic_ratio(launches)

    def roofline_of(ms, variant):
        ach = step_algo_bytes / (ms * 1e-3) / 1e9
        return {"bound": "hbm", "achieved": ach, "peak": hbm_peak, "unit": "GB/s", "frac": ach / hbm_peak,
                "traffic": step_algo_bytes * ratio if ratio else None, "traffic_note": ratio_note, "peak_kind": f"{peak_kind} copy bandwidth",
                "kernel": "qmv_mma_kernel (m <= 4 and the narrow shapes), qmv_tc_kernel + qmv_tc_pack_kernel, qmv_stream_kernel",
                "variant": variant, "ms_per_step": ms,
                "note": "achieved = (weight + activation + output bytes of the 32 mat-vecs) / event-timed step"}

    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": sweep_config(world),
        "run": {"launch": "CUDA graph replay" if graph is not None else "direct launches + NCCL all-gather per mat-vec",
                "exchange": "none" if world == 1 else ("peer stores from the mat-vec kernels into every rank's result "
                "buffer (symmetric memory) + one cross-rank barrier per step" if symm is not None else
                "NCCL all-gather per mat-vec")},
        "roofline": roofline_of(ms_chain if ms_chain is not None else ms_step,
                                "dependent chain: all 32 mat-vecs write one shared result buffer, each waits for the one ahead"
                                if ms_chain is not None else "independent launches (no chain variant on more than one GPU)"),
        "roofline_independent": roofline_of(ms_step, "independent launches: conflict-free neighbours overlap or leave as one kernel"),
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_s * 1e3, "steps_in_flight": e2e_in_flight},
        "gpu_launches": int(n_launch),
        "gpu_launches_chain": int(chain_launches) if chain_launches is not None else None,
        "clocks": clocks,
    }

    if world == 1:
        line["cpu_baseline"] = cpu_baseline()
        if not args.no_extra:
            try:
                line["extra"] = extra_numbers(mx, dev, reg, torch, tf_peak, hbm_peak)
                line["roofline_by_config"] = by_config(line["extra"], line["roofline_independent"],
                                                       line["roofline"] if ms_chain is not None else None, hbm_peak, tf_peak)
            except Exception as ex:  # the headline stands on its own
                line["extra"] = {"error": repr(ex)}
    if sharded is not None:
        line["extra"] = sharded
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()
    if sharded is not None and sharded.get("failed_checks"):
        raise SystemExit("multi-GPU correctness checks failed: " + "; ".join(sharded["failed_checks"]))


def sharded_extra(mx, dev, reg, torch, dist, rank, world, enc, ext_stream, pbar=None):
    """Secondary multi-GPU figures, every rank taking part:
    the expert-sharded MoE FFN layer (128 experts / world per rank, local routing filter, one all-reduce of the
    [T, hidden] partial sums as the combine) and the N-sharded Q6_K lm_head mat-vec (151936 x 5120, m = 1, peer
    stores into every rank's logits + one cross-rank barrier)."""
    from mlx_native_b200 import sharding
    from mlx_native_b200.ggml_pack import random_blocks

    out = {}
    failures = []                            # correctness checks that failed (reported at the end: every rank runs on)
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

    # ---- the same layer with tokens sharded too and all-to-all dispatch / combine (sharding.MoeAllToAll over NCCL):
    # ---- rank r owns T / world tokens and E / world experts; every (token, slot) row travels to its expert's rank,
    # ---- is computed there, and travels back unreduced, so the output is bit-identical to the one-GPU layer
    try:
        a2a = sharding.MoeAllToAll(E, top_k)
        moe2 = {}
        for T in (512, 1):
            logits = rng.standard_normal((T, E)).astype(np.float32)          # same on every rank
            xfull = rng.standard_normal((T, hidden)).astype(np.float32)
            t_lo, t_hi = T * rank // world, T * (rank + 1) // world
            Tl = t_hi - t_lo
            cap = T * top_k                                                   # every pair could land on one rank
            tz = lambda *shape, dt=torch.float32: torch.zeros(shape, dtype=dt, device="cuda")
            wrap = lambda t, dt: dev.wrap_device_memory(t.data_ptr(), max(t.numel(), 1) * t.element_size(), dt)
            x_t = torch.from_numpy(xfull[t_lo:t_hi].copy()).cuda() if Tl else tz(1, hidden)
            lg_t = torch.from_numpy(logits[t_lo:t_hi].copy()).cuda() if Tl else tz(1, E)
            ids_t, rw_t = tz(max(Tl, 1) * top_k, dt=torch.int32), tz(max(Tl, 1) * top_k)
            rows_t, lids_t = tz(cap, hidden), tz(cap, dt=torch.int32)
            yg_t, yu_t, act_t, yd_t = tz(cap, ffn), tz(cap, ffn), tz(cap, ffn), tz(cap, hidden)
            pairs_t, out_t = tz(max(Tl, 1) * top_k, hidden), tz(max(Tl, 1), hidden)
            lg_b, ids_b, rw_b = wrap(lg_t, mx.DType.F32), wrap(ids_t, mx.DType.U32), wrap(rw_t, mx.DType.F32)
            rows_b, lids_b = wrap(rows_t, mx.DType.F32), wrap(lids_t, mx.DType.U32)
            yg_b, yu_b, act_b, yd_b = (wrap(t, mx.DType.F32) for t in (yg_t, yu_t, act_t, yd_t))
            pairs_b, out_b = wrap(pairs_t, mx.DType.F32), wrap(out_t, mx.DType.F32)
            scratch = mx.IdMmScratch.alloc(dev, cnt, cap)

            def layer_a2a():
                if Tl:
                    mx.moe_softmax_topk(enc, reg, dev, lg_b, ids_b, rw_b, Tl, E, top_k)
                with torch.cuda.stream(torch.cuda.ExternalStream(enc.stream())):      # joins the encoder's lanes
                    plan = a2a.plan(ids_t[:Tl * top_k])
                    rows, lids = a2a.dispatch(plan, x_t[:Tl], rows_t, lids_t)
                P = rows.shape[0]
                if P:
                    pg2 = mx.GgmlQuantizedMatmulIdParams(P, 1, ffn, hidden, cnt, w["gate_stride"], mx.GgmlType.Q4_0)
                    pd2 = mx.GgmlQuantizedMatmulIdParams(P, 1, hidden, ffn, cnt, w["down_stride"], mx.GgmlType.Q6_K)
                    mx.quantized_matmul_id_ggml_pooled(enc, reg, dev, rows_b, w["gate"], lids_b, yg_b, scratch, pg2)
                    mx.quantized_matmul_id_ggml_pooled(enc, reg, dev, rows_b, w["up"], lids_b, yu_b, scratch, pg2)
                    mx.silu_mul(enc, reg, dev, yg_b, yu_b, act_b, P * ffn)
                    mx.quantized_matmul_id_ggml_pooled(enc, reg, dev, act_b, w["down"], lids_b, yd_b, scratch, pd2)
                with torch.cuda.stream(torch.cuda.ExternalStream(enc.stream())):
                    a2a.combine(plan, yd_t[:P], pairs_t[:Tl * top_k])
                if Tl:
                    mx.moe_weighted_reduce(enc, reg, dev, rw_b, pairs_b, out_b, Tl, top_k, hidden)

            sec = timed(layer_a2a)
            # bit-identity with the one-GPU layer: rank 0 holds every rank's experts and runs the whole layer alone
            gathered = [torch.empty((T * (r + 1) // world - T * r // world, hidden), dtype=torch.float32, device="cuda")
                        for r in range(world)]
            enc.commit_and_wait()
            torch.cuda.synchronize()
            dist.all_gather(gathered, out_t[:Tl].contiguous())
            identical = None
            if rank == 0:
                full = {}
                parts = {"gate": [], "up": [], "down": []}
                for r in range(world):
                    rr = np.random.default_rng(100 + r)               # same draw order as when the shards were made
                    for nm, tt, rws, cls in (("gate", "Q4_0", cnt * ffn, hidden), ("up", "Q4_0", cnt * ffn, hidden),
                                             ("down", "Q6_K", cnt * hidden, ffn)):
                        parts[nm].append(random_blocks(rr, tt, rws, cls))
                for name in parts:
                    allw = np.concatenate(parts[name])
                    full[name] = dev.alloc_buffer(allw.size, mx.DType.U8)
                    full[name].upload(allw)
                    full[name + "_stride"] = allw.size // E
                del parts
                e1 = dev.command_encoder()
                lg1, x1 = dev.alloc_buffer(logits.nbytes, mx.DType.F32), dev.alloc_buffer(xfull.nbytes, mx.DType.F32)
                lg1.upload(logits)
                x1.upload(xfull)
                ids1, rw1 = dev.alloc_buffer(T * top_k * 4, mx.DType.U32), dev.alloc_buffer(T * top_k * 4, mx.DType.F32)
                g1, u1, a1 = (dev.alloc_buffer(T * top_k * ffn * 4, mx.DType.F32) for _ in range(3))
                d1, o1 = dev.alloc_buffer(T * top_k * hidden * 4, mx.DType.F32), dev.alloc_buffer(T * hidden * 4, mx.DType.F32)
                pg1 = mx.GgmlQuantizedMatmulIdParams(T, top_k, ffn, hidden, E, full["gate_stride"], mx.GgmlType.Q4_0)
                pd1 = mx.GgmlQuantizedMatmulIdParams(T * top_k, 1, hidden, ffn, E, full["down_stride"], mx.GgmlType.Q6_K)
                mx.moe_softmax_topk(e1, reg, dev, lg1, ids1, rw1, T, E, top_k)
                mx.quantized_matmul_id_ggml(e1, reg, dev, x1, full["gate"], ids1, g1, pg1)
                mx.quantized_matmul_id_ggml(e1, reg, dev, x1, full["up"], ids1, u1, pg1)
                mx.silu_mul(e1, reg, dev, g1, u1, a1, T * top_k * ffn)
                mx.quantized_matmul_id_ggml(e1, reg, dev, a1, full["down"], ids1, d1, pd1)
                mx.moe_weighted_reduce(e1, reg, dev, rw1, d1, o1, T, top_k, hidden)
                e1.commit_and_wait()
                want = o1.download(np.float32).reshape(T, hidden)
                got = torch.cat(gathered, dim=0).cpu().numpy()
                identical = bool(np.array_equal(got.view(np.uint32), want.view(np.uint32)))
                rel = float(np.max(np.abs(got - want)) / max(float(np.max(np.abs(want))), 1e-30))
                if not identical:
                    # (recorded, not raised here: the other ranks are on their way into the next section's collectives)
                    failures.append(f"all-to-all MoE layer (T={T}) is not bit-identical to the one-GPU layer: "
                                    f"max |diff| / max |value| = {rel:.3e}")
                del full
            moe2[f"m{T}"] = {"tokens_per_s": T / sec, "ms_per_layer": sec * 1e3, "experts_per_rank": cnt,
                             "exchange": "NCCL all-to-all dispatch of (row, local expert id) per (token, slot) pair + all-to-all "
                                         "combine of the unreduced result rows", "bit_identical_to_one_gpu": identical,
                             "max_rel_diff_to_one_gpu": rel if rank == 0 else None}
        out["moe_ffn_layer_all_to_all"] = moe2
    except Exception as ex:
        out["moe_ffn_layer_all_to_all"] = {"error": repr(ex)}

    # ---- N-sharded lm_head, Q6_K 151936 x 5120: m = 1 (mat-vec) and m = 256 (mat-mat); every rank's kernels store their
    # ---- columns into all ranks' logits (peer stores from the kernels' epilogues) + one cross-rank barrier
    n, k = 151936, 5120
    try:
        from oracle import oracle as orc

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        n_loc = n // world
        rb = k // 256 * 210
        blk = random_blocks(wrng, "Q6_K", n_loc, k)
        wb = dev.alloc_buffer(blk.size, mx.DType.U8)
        wb.upload(blk)
        # rows of this rank that the oracle re-computes: first, second and last of the shard
        mine_rows = [0, 1, n_loc // 2, n_loc - 1]
        my_w = np.concatenate([blk[r * rb:(r + 1) * rb] for r in mine_rows])
        all_w = [None] * world
        dist.all_gather_object(all_w, my_w)
        chk_rows = [r * n_loc + i for r in range(world) for i in mine_rows]
        chk_w = np.concatenate(all_w)
        for m in (1, 256):
            x = rng.standard_normal((m, k)).astype(np.float32)              # same on every rank
            xb = dev.alloc_buffer(x.nbytes, mx.DType.F32, [m, k])
            xb.upload(x)
            buf = symm_mem.empty(m * n, dtype=torch.float32, device=f"cuda:{torch.cuda.current_device()}")
            hdl = symm_mem.rendezvous(buf, dist.group.WORLD)
            buf.zero_()
            ptrs = [int(p) for p in hdl.buffer_ptrs]
            yb = dev.wrap_device_memory(ptrs[rank], m * n * 4, mx.DType.F32, [m, n])
            peers = [ptrs[r] for r in range(world) if r != rank]
            prm = mx.GgmlQuantizedMatmulParams(m, n_loc, k, mx.GgmlType.Q6_K)

            if pbar is None:
                pbar = sharding.PeerBarrier(torch.cuda.current_device())

            def step():
                mx.quantized_matmul_ggml_sharded(enc, reg, dev, xb, wb, yb, prm, n, rank * n_loc, peers)
                pbar.wait(enc)

            sec = timed(step)
            got = buf.view(m, n)[:, chk_rows].cpu().numpy()
            ref, ad = orc.qmatmul(orc.Q6_K, chk_w, x, len(chk_rows), k, nthreads=4)
            err = float(np.max(np.abs(got.astype(np.float64) - ref) / np.maximum(ad, 1e-30)))
            tol = 1e-5 if m <= 8 else 2e-3
            if not err <= tol:
                raise RuntimeError(f"rank {rank}: sharded lm_head m={m} differs from the oracle: normalised error {err:.3e}")
            sent = m * n_loc * 4 * (world - 1)                                # bytes this rank stores to its peers
            out[f"lm_head_q6k_m{m}_n_sharded"] = {
                "us": sec * 1e6, "weight_GBps_all_ranks": n * rb / sec / 1e9, "tflops_all_ranks": 2.0 * m * n * k / sec / 1e12,
                "kernel": mx.last_kernel_name(), "oracle_norm_err": err,
                "nvlink_out_GBps_per_gpu": sent / sec / 1e9, "nvlink_frac_of_measured_770": sent / sec / 1e9 / 770.0,
                "nvlink_frac_of_nominal_900": sent / sec / 1e9 / 900.0,
                "exchange": "peer stores from the kernel epilogues + one barrier"}
            del buf, hdl
    except Exception as ex:
        out["lm_head_q6k_n_sharded"] = {"error": repr(ex)}
        if "differs from the oracle" in repr(ex):
            failures.append(repr(ex))                  # (the last section: no collective follows on the other ranks)
    if failures:
        out["failed_checks"] = failures
    return out


def reference_sample(sample_rows=128):
    """The bounded sample both CPU legs use: the whole sweep (8 (type, shape) pairs x m in {1, 2, 4, 8}) cut to
    `sample_rows` weight rows per mat-vec."""
    from oracle import oracle as orc

    otype = {"Q8_0": orc.Q8_0, "Q6_K": orc.Q6_K}
    rng = np.random.default_rng(0)
    items = []
    for t in TYPE_NAMES:
        for (n, k) in SHAPES:
            rows = min(n, sample_rows)
            wf = (rng.standard_normal((rows, k), dtype=np.float32) * np.float32(0.02))
            wq = orc.quantize(otype[t], wf, rule="ggml")
            for m in MS:
                items.append((otype[t], rows, k, wq, rng.standard_normal((m, k)).astype(np.float32)))
    return items, sum(w.size for (_, _, _, w, _) in items), sample_rows


def sweep_config(world=1, graph=True, symm=False):
    """`config` of the JSON line; the same for both arms."""
    return {"workload": "decode mat-vec sweep: Qwen3-8B projections (4096->4096, 4096->1024, 4096->12288, "
                        "12288->4096) x {Q8_0,Q6_K} x m in {1,2,4,8}; 32 mat-vecs per step",
            "weight_bytes_per_step": sum(weight_bytes(t, n, k) for t in TYPE_NAMES for (n, k) in SHAPES for _ in MS),
            "l2": "each launch has its own weight buffer: 915 MB of distinct weights per step, larger than L2",
            "parallelism": f"n-shard x{world}"}


def time_oracle(items, nthreads, steps, warmup=1):
    from oracle import oracle as orc

    def step():
        for (ot, rows, k, w, x) in items:
            orc.qmatmul(ot, w, x, rows, k, nthreads=nthreads, want_absdot=False)

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    return (time.perf_counter() - t0) / steps


def cpu_baseline():
    """The CPU oracle (kind "port": the upstream scalar path restated in C; the Rust reference cannot be built here) on
    the reference arm's sample, with all host threads and with one."""
    cores = os.cpu_count() or 1
    items, step_bytes, rows = reference_sample()
    t_all = time_oracle(items, cores, steps=20)
    t_one = time_oracle(items, 1, steps=3)
    return {"value": step_bytes / t_all / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
            "one_thread": {"value": step_bytes / t_one / 1e9, "unit": "GB/s", "cores": 1},
            "sample": f"the whole sweep cut to {rows} weight rows per mat-vec ({step_bytes / 1e6:.1f} MB of weights per "
                      f"pass); 20 passes on {cores} threads, 3 passes on 1 thread"}


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
    for (n, k, ms) in ((4096, 4096, (512, 2048)), (12288, 4096, (512, 2048)), (4096, 12288, (512, 2048))):
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
                mm[f"{t}_m{m}_n{n}_k{k}"] = {"tflops": tf, "ms": sec * 1e3, "frac_of_measured_bf16_peak": tf / tf_peak,
                                             "frac_of_nominal_2250": tf / 2250.0}
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

        pl = mx.MoeFfnLayerParams(T, top_k, hidden, ffn, E, mx.GgmlType.Q4_0, mx.GgmlType.Q4_0, mx.GgmlType.Q6_K, w1.size, w1.size, w2.size)

        def layer(e):
            # router, the expert half as one call (decode: routed mat-vecs for gate and up in one launch and the SwiGLU formed
            # on the down projection's activation load, as upstream's fused quantized_matmul_id_swiglu_q4_0 does,
            # src/ops/quantized_matmul_id_ggml.rs:551-670; prefill: one bucketing, one tile list and one activation pack
            # for gate and up, the SwiGLU formed while the down projection's operand is packed), weighted reduce
            mx.moe_softmax_topk(e, reg, dev, lg, ids, rw, T, E, top_k)
            mx.moe_ffn_layer(e, reg, dev, xb, ids, wg, wu, wd, yg, yu, yd, pl)
            mx.moe_weighted_reduce(e, reg, dev, rw, yd, outb, T, top_k, hidden)

        def layer_calls(e):
            # the same layer as the calls upstream's callers encode one by one
            mx.moe_softmax_topk(e, reg, dev, lg, ids, rw, T, E, top_k)
            mx.quantized_matmul_id_ggml(e, reg, dev, xb, wg, ids, yg, pg)
            mx.quantized_matmul_id_ggml(e, reg, dev, xb, wu, ids, yu, pg)
            mx.silu_mul(e, reg, dev, yg, yu, act, T * top_k * ffn)
            mx.quantized_matmul_id_ggml(e, reg, dev, act, wd, ids, yd, pd)
            mx.moe_weighted_reduce(e, reg, dev, rw, yd, outb, T, top_k, hidden)

        sec = timed(layer)
        sec_calls = timed(layer_calls)
        active = min(E, T * top_k)
        wbytes = active * (2 * w1.size + w2.size) if T == 1 else E * (2 * w1.size + w2.size)
        moe[f"m{T}"] = {"tokens_per_s": T / sec, "ms_per_layer": sec * 1e3, "expert_weight_GBps": wbytes / sec / 1e9,
                        "frac_of_measured_hbm_peak": wbytes / sec / 1e9 / hbm_peak, "ms_per_layer_call_by_call": sec_calls * 1e3}
    out["moe_ffn_layer"] = moe

    # lm_head: Q6_K 151936 x 5120 (638 MB), m = 1 (mat-vec, HBM-bound) and m = 256 (mat-mat)
    from mlx_native_b200.ggml_pack import random_blocks
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

    # configuration 1: Q4_0 4096 x 4096, m = 1; 16 weight copies (151 MB, more than L2) per replayed graph, once with
    # 16 result buffers (independent calls) and once with one (each call waits for the one ahead)
    n, k, copies = 4096, 4096, 16
    wq = gp.pack(gp.Q4_0, (rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)))
    wbs = []
    for _ in range(copies):
        b = dev.alloc_buffer(wq.size, mx.DType.U8)
        b.upload(wq)
        wbs.append(b)
    x = rng.standard_normal((1, k)).astype(np.float32)
    xb = dev.alloc_buffer(x.nbytes, mx.DType.F32)
    xb.upload(x)
    ys = [dev.alloc_buffer(n * 4, mx.DType.F32) for _ in range(copies)]
    p1 = mx.GgmlQuantizedMatmulParams(1, n, k, mx.GgmlType.Q4_0)
    c1 = {}
    for name, outs in (("independent", ys), ("chain", [ys[0]] * copies)):
        def seq(e, outs=outs):
            for wb_, yb_ in zip(wbs, outs):
                mx.quantized_matmul_ggml(e, reg, dev, xb, wb_, yb_, p1)
        sec = timed(seq, inner=1) / copies
        c1[name] = {"us": sec * 1e6, "weight_GBps": wq.size / sec / 1e9, "frac_of_measured_hbm_peak": wq.size / sec / 1e9 / hbm_peak}
    out["q4_0_4096x4096_m1"] = c1
    return out


def by_config(extra, sweep_indep, sweep_chain, hbm_peak, tf_peak):
    """One {bound, achieved, peak, frac, unit} entry per benchmark configuration and cell."""
    r = {}
    if "q4_0_4096x4096_m1" in extra:
        for name, v in extra["q4_0_4096x4096_m1"].items():
            r[f"config1 Q4_0 4096x4096 m=1 ({name})"] = {"bound": "hbm", "achieved": v["weight_GBps"], "peak": hbm_peak,
                                                       "frac": v["frac_of_measured_hbm_peak"], "unit": "GB/s", "us": v["us"]}
    r["config2 decode sweep (independent)"] = {k: sweep_indep[k] for k in ("bound", "achieved", "peak", "frac", "unit")}
    if sweep_chain is not None:
        r["config2 decode sweep (dependent chain)"] = {k: sweep_chain[k] for k in ("bound", "achieved", "peak", "frac", "unit")}
    for name, v in extra.get("qmm", {}).items():
        r[f"config3 {name}"] = {"bound": "tensor", "achieved": v["tflops"], "peak": tf_peak, "frac": v["frac_of_measured_bf16_peak"],
                                "frac_of_nominal_2250": v["frac_of_nominal_2250"], "unit": "TFLOP/s"}
    for name, v in extra.get("moe_ffn_layer", {}).items():
        r[f"config4 MoE FFN layer {name}"] = {"bound": "hbm", "achieved": v["expert_weight_GBps"], "peak": hbm_peak,
                                             "frac": v["frac_of_measured_hbm_peak"], "unit": "GB/s",
                                             "tokens_per_s": v["tokens_per_s"], "ms_per_layer": v["ms_per_layer"]}
    lm = extra.get("lm_head_q6k", {})
    if "m1" in lm:
        r["config5 lm_head Q6_K m=1"] = {"bound": "hbm", "achieved": lm["m1"]["weight_GBps"], "peak": hbm_peak,
                                        "frac": lm["m1"]["frac_of_measured_hbm_peak"], "unit": "GB/s", "us": lm["m1"]["us"]}
    if "m256" in lm:
        r["config5 lm_head Q6_K m=256"] = {"bound": "tensor", "achieved": lm["m256"]["tflops"], "peak": tf_peak,
                                          "frac": lm["m256"]["tflops"] / tf_peak, "frac_of_nominal_2250": lm["m256"]["tflops"] / 2250.0,
                                          "unit": "TFLOP/s", "us": lm["m256"]["us"]}
    return r


# --------------------------------------------------------------------------------------------- profiler workloads
def run_case(argv):
    """Small fixed workloads for profiler captures (a few hundred MB on the device, a handful of launches).

      --case mv  [Q8_0|Q6_K|Q4_0] [m]   decode mat-vec, n=12288 k=4096, 4 weight copies (> L2), two passes
      --case mvs [Q8_0|Q6_K|Q4_0] [m]   the same on the narrow shape n=1024 k=4096, 40 weight copies (> L2)
      --case mm  [Q4_0|Q6_K|Q8_0] [m]   prefill mat-mat, n=4096 k=4096, m=512 by default
      --case moe [m]                    expert-routed gate projection, 128 experts, top-8
      --case moe_layer [m] [reps] [calls]  whole MoE FFN layer (router, moe_ffn_layer, reduce; `calls`: the expert half call by call), 128 experts, top-8
      --case moe_trace [gate|down]      cycle trace of one CTA of the grouped mat-mat (experiment build only)
      --case cmp [types] [ms]           the mat-vec kernels side by side, microseconds per call, independent and chained
                                        (CUDA-graph replay over rotating weight copies > L2)
      --case gap                        microseconds per launch of a chain of dependent trivial kernels
    The kernel variant follows the MLXN_QMV / MLXN_QMM environment variables.  Weights are random bytes with finite
    f16 scales: the kernels' timing and memory traffic do not depend on the values."""
    import mlx_native_b200 as mx
    from mlx_native_b200.ggml_pack import random_blocks

    gt = {"Q4_0": mx.GgmlType.Q4_0, "Q8_0": mx.GgmlType.Q8_0, "Q6_K": mx.GgmlType.Q6_K, "Q4_K": mx.GgmlType.Q4_K}
    mode = argv[0] if argv else "mv"
    dev = mx.MlxDevice.new(0)
    reg = mx.KernelRegistry.new()
    rng = np.random.default_rng(0)

    def upload(a, dt=mx.DType.U8):
        b = dev.alloc_buffer(a.nbytes, dt)
        b.upload(a)
        return b

    if mode == "cmp":
        types = (argv[1] if len(argv) > 1 else "Q8_0,Q6_K,Q4_0").split(",")
        ms = [int(v) for v in (argv[2] if len(argv) > 2 else "1,2,4,8").split(",")]

        def timed(t, n, k, m, variant, chain, reps=10):
            wbytes = weight_bytes(t, n, k)
            ncopies = int(max(4, min(48, (300e6 // wbytes) + 1)))
            w = random_blocks(rng, t, n, k)
            ws = [upload(w) for _ in range(ncopies)]
            xb = upload(rng.standard_normal((m, k)).astype(np.float32), mx.DType.F32)
            ys = [dev.alloc_buffer(m * n * 4, mx.DType.F32) for _ in range(1 if chain else ncopies)] * (ncopies if chain else 1)
            p = mx.GgmlQuantizedMatmulParams(m, n, k, gt[t])
            mx.set_option("qmv", variant)
            enc = dev.command_encoder()
            for wb, yb in zip(ws[:2], ys[:2]):
                mx.quantized_matmul_ggml(enc, reg, dev, xb, wb, yb, p)
            enc.commit_and_wait()
            enc.begin_capture()
            for wb, yb in zip(ws, ys):
                mx.quantized_matmul_ggml(enc, reg, dev, xb, wb, yb, p)
            g = enc.end_capture()
            for _ in range(2):
                g.launch(enc)
            enc.commit_and_wait()
            for _ in range(reps):
                g.launch(enc)
            return enc.commit_wait_with_gpu_time() / (reps * ncopies) * 1e6

        for t in types:
            for (n, k) in SHAPES:
                for m in ms:
                    ideal = weight_bytes(t, n, k) / (measured_peaks()[0] * 1e3)
                    variants = ("auto", "simple") if t == "Q4_K" else ("auto", "mma", "tc", "stream")
                    cells = [f"{v}{'/chain' if ch else ''} {timed(t, n, k, m, v, ch):6.2f}"
                             for ch in (False, True) for v in variants if not (v in ("stream", "simple") and m > 2)]
                    print(f"{t} {n:6d}x{k:<6d} m={m} ideal {ideal:5.2f} us | " + " ".join(cells), flush=True)
        mx.set_option("qmv", "auto")
        return
    if mode == "gap":
        # what a dependent launch costs on this device whatever it computes: chains of kernels that each wait for the
        # one before (CUDA-graph replay, device-timed) -- a 64-element SwiGLU (ordinary launches) and a 16 x 256 mat-vec
        # of the register-level kernel (programmatic dependent launches)
        n_el, reps, chain_len = 64, 10, 200
        a = upload(rng.standard_normal(n_el).astype(np.float32), mx.DType.F32)
        b = upload(rng.standard_normal(n_el).astype(np.float32), mx.DType.F32)
        w = upload(random_blocks(rng, "Q8_0", 16, 256))
        xs = [upload(rng.standard_normal(256).astype(np.float32), mx.DType.F32)]
        y = dev.alloc_buffer(16 * 4, mx.DType.F32)
        p = mx.GgmlQuantizedMatmulParams(1, 16, 256, mx.GgmlType.Q8_0)
        mx.set_option("qmv", "mma")

        def chain(kind, e):
            for _ in range(chain_len):
                if kind == "plain":
                    mx.silu_mul(e, reg, dev, a, b, a, n_el)
                else:
                    mx.quantized_matmul_ggml(e, reg, dev, xs[0], w, y, p)   # the same result buffer: write after write

        for kind in ("plain", "overlapped"):
            enc = dev.command_encoder()
            chain(kind, enc)
            enc.commit_and_wait()
            enc.begin_capture()
            chain(kind, enc)
            g = enc.end_capture()
            g.launch(enc)
            enc.commit_and_wait()
            for _ in range(reps):
                g.launch(enc)
            us = enc.commit_wait_with_gpu_time() / (reps * chain_len) * 1e6
            print(f"dependent launch, {kind}: {us:.2f} us per kernel")
        mx.set_option("qmv", "auto")
        return
    enc = dev.command_encoder()
    E, top_k, hidden, ffn = 128, 8, 2048, 768
    if mode == "moe_layer":
        T = int(argv[1]) if len(argv) > 1 else 512
        reps = int(argv[2]) if len(argv) > 2 else 3
        bufs = {}
        for name, t, rows, cols in (("gate", "Q4_0", E * ffn, hidden), ("up", "Q4_0", E * ffn, hidden), ("down", "Q6_K", E * hidden, ffn)):
            w = random_blocks(rng, t, rows, cols)
            bufs[name] = upload(w)
            bufs[name + "_stride"] = w.size // E
        lg = upload(rng.standard_normal((T, E)).astype(np.float32), mx.DType.F32)
        xb = upload(rng.standard_normal((T, hidden)).astype(np.float32), mx.DType.F32)
        ids = dev.alloc_buffer(T * top_k * 4, mx.DType.U32)
        rw = dev.alloc_buffer(T * top_k * 4, mx.DType.F32)
        yg, yu, act = (dev.alloc_buffer(T * top_k * ffn * 4, mx.DType.F32) for _ in range(3))
        yd = dev.alloc_buffer(T * top_k * hidden * 4, mx.DType.F32)
        outb = dev.alloc_buffer(T * hidden * 4, mx.DType.F32)
        pg = mx.GgmlQuantizedMatmulIdParams(T, top_k, ffn, hidden, E, bufs["gate_stride"], mx.GgmlType.Q4_0)
        pd = mx.GgmlQuantizedMatmulIdParams(T * top_k, 1, hidden, ffn, E, bufs["down_stride"], mx.GgmlType.Q6_K)
        calls = len(argv) > 3 and argv[3] == "calls"      # the layer call by call instead of as one moe_ffn_layer call
        pl = mx.MoeFfnLayerParams(T, top_k, hidden, ffn, E, mx.GgmlType.Q4_0, mx.GgmlType.Q4_0, mx.GgmlType.Q6_K,
                                  bufs["gate_stride"], bufs["up_stride"], bufs["down_stride"])
        for _ in range(reps):
            mx.moe_softmax_topk(enc, reg, dev, lg, ids, rw, T, E, top_k)
            if not calls:
                mx.moe_ffn_layer(enc, reg, dev, xb, ids, bufs["gate"], bufs["up"], bufs["down"], yg, yu, yd, pl)
            else:
                mx.quantized_matmul_id_ggml(enc, reg, dev, xb, bufs["gate"], ids, yg, pg)
                mx.quantized_matmul_id_ggml(enc, reg, dev, xb, bufs["up"], ids, yu, pg)
                mx.silu_mul(enc, reg, dev, yg, yu, act, T * top_k * ffn)
                mx.quantized_matmul_id_ggml(enc, reg, dev, act, bufs["down"], ids, yd, pd)
            mx.moe_weighted_reduce(enc, reg, dev, rw, yd, outb, T, top_k, hidden)
            enc.commit_and_wait()
        print("ok", mx.last_kernel_name())
        return
    if mode == "moe_trace":
        # cycle trace of CTA 0 of the grouped mat-mat (gate: Q4_0 768 x 2048 per expert; down: Q6_K 2048 x 768), T = 512.
        # Needs a library built with MLXN_NVCC_EXTRA="-DMLXN_EXPERIMENTS -DMLXN_TC_TRACE" and MLXN_TC_DEBUG=768 in the
        # environment (the kernel then logs (event, clock) pairs into the result buffer instead of writing results).
        # Prints "cycles role event index" lines: roles wprod (weight copies: 1 = stage requested), mma0 / mma1 (1 = item
        # start, 2 = weights of a stage ready, 4 = activations ready, 5 = MMAs issued, 3 = committed), dq0 / dq1 (the two
        # sets of dequantising warps: 1 = item start, 2 = raw stage arrived, 3 = ring place free, 8 = dequantised,
        # 9 = stored to tensor memory, 4 = handed to the MMA warp, 10 = raw stage released, 5 / 6 / 7 = read-back).
        which = argv[1] if len(argv) > 1 else "gate"
        T = 512
        t, n, k, m, tk = ("Q4_0", ffn, hidden, T, top_k) if which == "gate" else ("Q6_K", hidden, ffn, T * top_k, 1)
        w = random_blocks(rng, t, E * n, k)
        wb = upload(w)
        xb = upload(rng.standard_normal((m, k)).astype(np.float32), mx.DType.F32)
        ib = upload(np.stack([rng.permutation(E)[:top_k] for _ in range(T)]).astype(np.uint32).reshape(-1), mx.DType.U32)
        yb = dev.alloc_buffer(m * tk * n * 4, mx.DType.F32)
        p = mx.GgmlQuantizedMatmulIdParams(m, tk, n, k, E, w.size // E, gt[t])
        for _ in range(2):
            mx.quantized_matmul_id_ggml(enc, reg, dev, xb, wb, ib, yb, p)
            enc.commit_and_wait()
        yb.upload(np.zeros(m * tk * n, np.float32))
        mx.quantized_matmul_id_ggml(enc, reg, dev, xb, wb, ib, yb, p)
        enc.commit_and_wait()
        tr = yb.download(np.float32).view(np.uint32)[:6 * 1024].reshape(6, 512, 2)
        ev = []
        for role, nm in {0: "wprod", 1: "mma0", 4: "mma1", 2: "dq0", 3: "dq1"}.items():
            for code_x, clk in tr[role]:
                if code_x == 0 and clk == 0:
                    break
                ev.append((int(clk), nm, int(code_x) >> 16, int(code_x) & 0xFFFF))
        if not ev:
            print("no trace events: the library was not built with -DMLXN_TC_TRACE, or MLXN_TC_DEBUG=768 is not set")
            return
        ev.sort(key=lambda e_: e_[0])
        for clk, nm, code, idx in ev:
            print(f"{(clk - ev[0][0]) & 0xFFFFFFFF:9d} {nm} {code} {idx}")
        return
    if mode == "moe":
        m = int(argv[1]) if len(argv) > 1 else 512
        w = random_blocks(rng, "Q4_0", E * ffn, hidden)
        wb = upload(w)
        xb = upload(rng.standard_normal((m, hidden)).astype(np.float32), mx.DType.F32)
        ib = upload(np.stack([rng.permutation(E)[:top_k] for _ in range(m)]).astype(np.uint32), mx.DType.U32)
        yb = dev.alloc_buffer(m * top_k * ffn * 4, mx.DType.F32)
        p = mx.GgmlQuantizedMatmulIdParams(m, top_k, ffn, hidden, E, w.size // E, mx.GgmlType.Q4_0)
        for _ in range(3):
            mx.quantized_matmul_id_ggml(enc, reg, dev, xb, wb, ib, yb, p)
        enc.commit_and_wait()
        print("ok", mx.last_kernel_name())
        return
    t = argv[1] if len(argv) > 1 else ("Q4_0" if mode == "mm" else "Q8_0")
    if mode == "mv":
        n, k, m, copies = 12288, 4096, int(argv[2]) if len(argv) > 2 else 1, 4
    elif mode == "mvs":
        n, k, m, copies = 1024, 4096, int(argv[2]) if len(argv) > 2 else 1, 40
    else:
        n, k, m, copies = 4096, 4096, int(argv[2]) if len(argv) > 2 else 512, 1
    w = random_blocks(rng, t, n, k)
    ws = [upload(w) for _ in range(copies)]
    xb = upload(rng.standard_normal((m, k)).astype(np.float32), mx.DType.F32)
    ys = [dev.alloc_buffer(m * n * 4, mx.DType.F32) for _ in range(copies)]
    p = mx.GgmlQuantizedMatmulParams(m, n, k, gt[t])
    for _ in range(2):
        for wbuf, yb in zip(ws, ys):
            mx.quantized_matmul_ggml(enc, reg, dev, xb, wbuf, yb, p)
        enc.commit_and_wait()
    print("ok", mx.last_kernel_name(), "launches", mx.kernel_launch_count())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip the secondary mat-mat / MoE figures")
    ap.add_argument("--case", nargs=argparse.REMAINDER, help="run one profiler workload instead of the benchmark (see run_case)")
    args = ap.parse_args()
    if args.case is not None:
        run_case(args.case)
        return
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
