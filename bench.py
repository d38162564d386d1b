"""Benchmark of the paged KV decode path on the MoE-decoder configuration.

Workload (one "step"): one decode token for each of 64 sequences through 48 layers — per
layer, append the step's K/V rows to the block pool (KV append) and run paged decode attention
over the whole context (bf16 KV, 32 query / 4 KV heads of 128, 16-position blocks scattered
over the pool by a seeded permutation, contexts uniform in [1024, 4096]).  Synthetic data.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

With N > 1 (under torchrun) every rank runs the same workload on its own sequences (the path
partitions by sequence: no collective in it), `value` is all ranks' tokens over the slowest
rank's time, scaling "weak".

One JSON line on stdout:
  value      tokens/s with every input already in device memory (one launch per layer: append fused
             into attention).  The K steps are timed as one block; the block is repeated until the
             timed region lasts at least a second, so the clock record holds tens of samples.  The
             block tables and work lists of every step are built and uploaded (qvx_tables_create)
             before the clock starts: `value` does not pay for them, `e2e` does.
  e2e        tokens/s through the host-memory call of the C ABI the reference's runtime would make:
             one synchronous qvx_paged_attention_host per layer (DiscreteDevice::routed_moe is complete
             on return, and layer l + 1's query does not exist before layer l has returned), pinned
             host buffers in, outputs back to the host, copies inside the timed region.
             `e2e.pipelined` is the same step through qvx_paged_attention_host_async x layers and one
             qvx_wait: what a caller that has all the layers' inputs at hand could reach.
  roofline   the attention kernel's algorithmic bytes per launch over its mean duration in the timed
             region (nothing else runs there), against the measured copy bandwidth of
             MEASURED_PEAKS.json
  parity_sample  one (sequence, layer) of the last timed step, read back with its blocks of the
             pool and checked against the CPU oracle after the clock has stopped
  cpu_baseline  the CPU restatement of the reference's own path, timed on this host (rank 0, N = 1)

--impl reference times only that CPU path, on all host threads, as the reference arm.
"""
from __future__ import annotations

import argparse
import ctypes as C
import dataclasses
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from qubivex_b200 import workload as wl  # noqa: E402

METRIC = "paged_kv_decode_tokens_per_s"
UNIT = "tokens/s"
SEED = 20261125
# dram__bytes_read.sum + dram__bytes_write.sum of one attention launch over its algorithmic
# bytes, from the ncu capture summarised in profiles/ (one layer of this workload).
DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE = 1.012


def env_int(name: str, default: int) -> int:
    return int(os.environ.get(name, default))


def bind_near_gpu(local_rank: int) -> str:
    """One process per GPU: keeps this process's threads -- and with them the pinned host buffers it is about
    to allocate and touch -- on the cores next to its GPU (the affinity NVML reports for the device, within
    what the process is allowed), so that eight ranks' host copies do not cross between sockets.  Changes nothing
    of the GPU; returns what was done, for the JSON line."""
    try:
        import pynvml
        import torch
        pynvml.nvmlInit()
        try:
            pr = torch.cuda.get_device_properties(local_rank)
            bus = f"{pr.pci_domain_id:08x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
            h = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
        except Exception:
            h = pynvml.nvmlDeviceGetHandleByIndex(local_rank)
        allowed = os.sched_getaffinity(0)
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (max(allowed) + 64) // 64)
        near = {64 * w + b for w, bits in enumerate(words) for b in range(64) if (int(bits) >> b) & 1}
        mine = near & allowed
        memory = prefer_memory_near_gpu(pynvml, h)
        if not mine or mine == allowed:
            return f"cores unchanged ({len(allowed)} allowed, {len(mine)} of them next to the GPU); {memory}"
        os.sched_setaffinity(0, mine)
        return f"{len(mine)} of {len(allowed)} allowed cores: those next to the GPU; {memory}"
    except Exception as e:  # no NVML, an old torch, a restricted container: the run goes on unbound
        return f"unchanged ({type(e).__name__})"


def prefer_memory_near_gpu(pynvml, handle) -> str:
    """The process's memory policy: prefer the NUMA node the GPU hangs off (what `numactl --preferred` does), so that
    the page-locked buffers allocated from here on are on that node even when the cores the container allows are on
    the other socket -- a rank whose copies cross the sockets' link shares it with every other such rank."""
    import ctypes
    try:
        words = pynvml.nvmlDeviceGetMemoryAffinity(handle, 1, pynvml.NVML_AFFINITY_SCOPE_NODE)
        mask = int(words[0])
        if not mask:
            return "memory policy unchanged (no node reported)"
        node = (mask & -mask).bit_length() - 1
        libc = ctypes.CDLL(None, use_errno=True)
        nodemask = ctypes.c_ulong(1 << node)
        SYS_set_mempolicy, MPOL_PREFERRED = 238, 1       # x86-64
        if os.uname().machine != "x86_64":
            return "memory policy unchanged (not x86-64)"
        rc = libc.syscall(SYS_set_mempolicy, MPOL_PREFERRED, ctypes.byref(nodemask), 65)
        if rc != 0:
            return f"memory policy unchanged (set_mempolicy: errno {ctypes.get_errno()})"
        return f"memory preferred on node {node}"
    except Exception as e:
        return f"memory policy unchanged ({type(e).__name__})"


def config_of(shape: "wl.Shape", layers: int) -> dict:
    """The workload's description: the same keys and values in both arms."""
    return {"workload": shape.name, "layers": layers, "batch_per_gpu": shape.batch, "heads": shape.heads,
            "kv_heads": shape.kv_heads, "head_dim": shape.head_dim, "block_tokens": shape.block_tokens,
            "context": [shape.ctx_lo, shape.ctx_hi], "partition": "by sequence, no collective",
            "l2": "each launch reads more than 300 MiB of KV, once (the L2 holds 126 MB): no flush between iterations"}


def measured_peak_gbs() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [x.strip() for x in line.split(",")]))

    def stop(self, t_from: float, t_to: float) -> dict:
        """Samples read between t_from and t_to (perf_counter: the device was under load then); all of
        them if the interval was too short to catch one."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        inside = [r for t, r in self.rows if t_from <= t <= t_to]
        rows = inside or [r for _, r in self.rows]
        sm = [float(r[0]) for r in rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active" for r in rows)]
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm), "samples_under_load": len(inside)}


# ---------------------------------------------------------------------------------------------
class CpuSample:
    """The CPU restatement of the reference's path (one task per (token, head) reading the paged
    pool, as its host path does) on a sample of the workload: `n` sequences x 1 layer x 1 decode
    step.  The pool is made once, for the longest contexts the run will ask for."""

    def __init__(self, shape: wl.Shape, lengths: np.ndarray, grow: int, threads: int, seed: int):
        import oracle

        self.oracle, self.shape, self.threads = oracle, shape, threads
        self.n = min(len(lengths), 16)
        self.base = np.asarray(lengths[:self.n], dtype=np.int64)
        B = shape.block_tokens
        self.geo = oracle.geometry(B, shape.kv_heads, shape.head_dim, oracle.BF16, oracle.LAYOUT_NATIVE)
        nb = int(((self.base + grow + 1 + B - 1) // B).sum())
        self.rng = np.random.default_rng([seed, 0x77])
        self.perm = self.rng.permutation(nb + 8).astype(np.uint32)
        scale = wl.value_scale(shape)
        self.pool = oracle.narrow(wl.normal(self.rng, ((nb + 8) * oracle.block_bytes(self.geo) // 2,), scale), oracle.BF16).view(np.uint8)
        self.q = wl.normal(self.rng, (self.n, shape.heads, shape.head_dim), scale)
        tabs = wl.tables_for(self.base + 1, B, self.perm)
        oracle.attn_decode(self.pool, self.geo, shape.heads, self.q[:1], tabs.pos[:1], tabs.blocks, tabs.table_at[:1], threads=threads)  # warm

    def run(self, step: int, target_s: float):
        """Contexts `step` positions on; repeated until about `target_s` of wall time.  Returns (seconds per
        sequence-layer, text)."""
        lens = self.base + step + 1
        tabs = wl.tables_for(lens, self.shape.block_tokens, self.perm)
        reps, t0 = 0, time.perf_counter()
        while True:
            rc, _ = self.oracle.attn_decode(self.pool, self.geo, self.shape.heads, self.q, tabs.pos, tabs.blocks, tabs.table_at,
                                            threads=self.threads)
            assert rc == 0
            reps += 1
            dt = time.perf_counter() - t0
            if dt >= target_s or reps >= 4096:
                break
        text = (f"{self.n} of the {self.shape.batch} sequences (contexts {int(lens.min())}-{int(lens.max())}) x 1 of the "
                f"{self.shape.layers} layers x 1 decode step, repeated {reps}x ({dt:.1f} s) on {self.threads} threads, one task per "
                f"(token, KV head): its rows gathered from the paged pool once, then attend per query head; "
                f"extrapolated: tokens/s = 1 / ({self.shape.layers} layers x seconds per sequence-layer), "
                f"i.e. the sample is 1/{self.shape.batch // self.n} of the batch x 1/{self.shape.layers} of the layers of a step")
        return dt / (reps * self.n), text


    def run_one_thread(self, step: int, target_s: float):
        """The device simulation's order on one thread (per token: gather the KV head's rows, then attend per query
        head, crates/qubivex-backend-cpu/src/sim.rs:404-428) on the first two sequences of the sample."""
        n = min(2, self.n)
        lens = self.base[:n] + step + 1
        tabs = wl.tables_for(lens, self.shape.block_tokens, self.perm)
        reps, t0 = 0, time.perf_counter()
        while True:
            rc, _ = self.oracle.attn_decode(self.pool, self.geo, self.shape.heads, self.q[:n], tabs.pos, tabs.blocks, tabs.table_at)
            assert rc == 0
            reps += 1
            dt = time.perf_counter() - t0
            if dt >= target_s or reps >= 4096:
                break
        return dt / (reps * n), f"{n} sequences (contexts {int(lens.min())}-{int(lens.max())}) x 1 layer x 1 step, repeated {reps}x ({dt:.1f} s), 1 thread"


def run_reference(args, rank: int, world: int) -> None:
    """The reference arm: the reference's CPU path (its C restatement: the Rust original cannot
    be built here) on all host threads, same metric and config, a bounded sample per step."""
    if rank != 0:
        return
    shape = wl.C2
    lengths = wl.contexts(shape, SEED)
    threads = os.cpu_count() or 1
    per = []
    total = args.warmup + args.steps
    sample = CpuSample(shape, lengths, total, threads, SEED)
    for i in range(total):
        sec, text = sample.run(i, target_s=max(0.5, 60.0 / max(total, 1)))  # the whole run: about a minute of timed work
        if i >= args.warmup:
            per.append(sec)
    sec = float(np.mean(per))
    value = 1.0 / (shape.layers * sec)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": shape.batch / value * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config_of(shape, shape.layers),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": text},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
def parity_sample(dev, pool, geo, shape, lengths, blocks, table_at, q_dev, out_dev, seq: int) -> dict:
    """Sequence `seq` of the last launch of the timed region against the CPU oracle: its blocks of the
    pool are read back (they hold the row the launch appended), the oracle attends over them with the
    launch's query, and the launch's output for the sequence must be within the 16-bit tolerance."""
    import oracle

    B = shape.block_tokens
    n = int(lengths[seq]) + 1                      # positions 0..=pos
    ids = blocks[int(table_at[seq]):int(table_at[seq]) + (n + B - 1) // B]
    geo_o = oracle.geometry(B, shape.kv_heads, shape.head_dim, oracle.BF16, oracle.LAYOUT_NATIVE)
    bb = oracle.block_bytes(geo_o)
    host_pool = np.concatenate([dev.read(pool, int(b) * bb, bb) for b in ids])
    q1 = q_dev[seq:seq + 1].cpu().numpy()
    rc, want = oracle.attn_decode(host_pool, geo_o, shape.heads, q1, np.array([n - 1], dtype=np.uint32),
                                  np.arange(len(ids), dtype=np.uint32), np.zeros(1, dtype=np.uint32), threads=os.cpu_count() or 1)
    got = out_dev[seq].cpu().numpy()
    err = np.abs(got.astype(np.float64) - want[0].astype(np.float64))
    ok = rc == 0 and bool(np.all(err <= 2e-3 + 1e-2 * np.abs(want[0])))
    return {"sequence": int(seq), "layer": "last", "positions": n, "max_abs_err": float(err.max()),
            "max_abs_oracle": float(np.abs(want[0]).max()), "max_err_over_allowed": float((err / (2e-3 + 1e-2 * np.abs(want[0]))).max()),
            "tolerance": "2e-3 + 1e-2 * |oracle|", "ok": ok}


def run_ours(args, rank: int, local_rank: int, world: int) -> None:
    import torch

    from qubivex_b200 import device as qd
    from qubivex_b200.device import ptr

    torch.cuda.set_device(local_rank)
    dist = None
    host_cores = "unchanged (one process)"
    if world > 1:
        host_cores = bind_near_gpu(local_rank)
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    sampler = ClockSampler(local_rank)  # runs from here on (its start-up takes longer than a short timed region)
    sampler.start()
    # CUDA events around every 64th launch of each kernel: a bracketed launch cannot overlap its neighbours'
    # ends, so bracketing every 4th cost the timed region 5 %; one in 64 still gives the launch-alone figure.
    dev = qd.CudaDevice(local_rank, timing=64)
    lib = dev.lib
    shape = wl.C2
    layers = args.layers or shape.layers
    s, d, heads, kvh, B = shape.batch, shape.head_dim, shape.heads, shape.kv_heads, shape.block_tokens
    kv_out = kvh * d
    geo = qd.geometry(B, kvh, d, qd.BF16, qd.LAYOUT_NATIVE)
    bb = qd.block_bytes(geo)
    scale = wl.value_scale(shape)
    W, K = args.warmup, args.steps
    We, Ke = min(W, 3), K
    total_steps = W + K + We + Ke
    # Every rank draws the same context lengths (so every GPU has the same number of bytes to move and
    # the max over ranks measures the machines, not the luck of the draw); its values and its block
    # placement are its own.
    lengths = wl.contexts(shape, SEED)                   # positions prefilled per sequence
    nb_seq = (lengths + total_steps + B - 1) // B          # table entries per sequence, with room to grow
    blocks_per_layer = int(nb_seq.sum())
    pool_blocks = blocks_per_layer * layers
    perm = wl.permutation(pool_blocks, SEED + rank)
    pool = dev.alloc(pool_blocks * bb)
    table_at = np.zeros(s, dtype=np.uint32)
    table_at[1:] = np.cumsum(nb_seq)[:-1]
    layer_blocks = [perm[l * blocks_per_layer:(l + 1) * blocks_per_layer].copy() for l in range(layers)]
    stream = torch.cuda.current_stream().cuda_stream
    gen = torch.Generator(device="cuda").manual_seed(SEED + rank)

    # ---- prefill through the sync path: every context row of every layer --------------------------
    seq_of = np.repeat(np.arange(s), lengths)
    pos_of = np.concatenate([np.arange(n) for n in lengths])
    n_rows = len(seq_of)
    chunk = 1 << 16
    for l in range(layers):
        blk = layer_blocks[l][table_at[seq_of] + pos_of // B].astype(np.int64)
        sync_to = torch.from_numpy((blk * B + pos_of % B).astype(np.uint32).view(np.int32)).cuda()
        for lo in range(0, n_rows, chunk):
            hi = min(n_rows, lo + chunk)
            rows = torch.randn((hi - lo, 2 * kv_out), device="cuda", dtype=torch.float32, generator=gen) * scale
            dev.check(lib.qvx_kv_sync(dev.h, C.byref(geo), C.c_void_p(pool.ptr), pool_blocks, ptr(rows), C.c_void_p(sync_to[lo:hi].data_ptr()),
                                      hi - lo, C.c_void_p(stream)))
        torch.cuda.synchronize()
    del sync_to, rows

    def tables_for_step(t: int, l: int):
        pos = (lengths + t).astype(np.uint32)
        out = C.c_void_p()
        dev.check(lib.qvx_tables_create(dev.h, C.byref(geo), pool_blocks, heads, s, ptr(pos), ptr(layer_blocks[l]), blocks_per_layer,
                                        ptr(table_at), C.byref(out)))
        return out

    # ---- value: everything resident ---------------------------------------------------------------
    tabs = [[tables_for_step(t, l) for l in range(layers)] for t in range(W + K)]
    q = [torch.randn((s, heads, d), device="cuda", generator=gen) * scale for _ in range(W + K)]
    kn = [torch.randn((s, kv_out), device="cuda", generator=gen) * scale for _ in range(W + K)]
    vn = [torch.randn((s, kv_out), device="cuda", generator=gen) * scale for _ in range(W + K)]
    out = torch.empty((s, heads, d), device="cuda")
    pool_p, sp = C.c_void_p(pool.ptr), C.c_void_p(stream)

    # Consecutive launches serve different layers, whose blocks are disjoint: the next layer's old
    # positions may start streaming while this layer's launch drains (its q, k_new and v_new still
    # wait for everything before it in the stream).
    variant = qd.ATTN_AUTO | (qd.ATTN_POOL_SETTLED if layers >= 2 else 0)

    def step(t: int):
        for l in range(layers):
            tb = tabs[t][l]
            # the step's append and its attention: one launch (the rows are stored by the CTAs that read them)
            dev.check(lib.qvx_kv_append_attn_decode(dev.h, tb, pool_p, ptr(kn[t]), ptr(vn[t]), ptr(q[t]), ptr(out), variant, sp))

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    for t in range(W):
        step(t)
    barrier()
    # One untimed block of the K steps tells how many repeats of the block make a second.
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record()
    for t in range(W, W + K):
        step(t)
    p1.record()
    barrier()
    pilot_ms = p0.elapsed_time(p1)
    repeats = torch.tensor([max(1, int(np.ceil(args.min_seconds * 1e3 / max(pilot_ms, 1e-3))))], device="cuda")
    if dist is not None:
        dist.all_reduce(repeats, op=dist.ReduceOp.MAX)
    R = int(repeats.item())
    dev.reset_kernel_times()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_load0 = time.perf_counter()
    e0.record()
    for _ in range(R):  # the K steps again: the same rows land on the same positions, the pool does not change
        for t in range(W, W + K):
            step(t)
    e1.record()
    barrier()
    clocks = sampler.stop(t_load0, time.perf_counter())
    ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    if dist is not None:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_total = float(ms.item()) / R      # per block of K steps
    kt = dev.kernel_times()
    value = world * s * K / (ms_total / 1e3)
    attn_launches, attn_ns = kt["attn"]
    parity = parity_sample(dev, pool, geo, shape, lengths + (W + K - 1), layer_blocks[layers - 1], table_at, q[W + K - 1], out,
                           SEED % s)
    algo = float(np.mean([wl.algorithmic_bytes(shape, lengths + t + 1) for t in range(W, W + K)]))
    # The timed region holds nothing but this kernel's launches, back to back on one stream: its
    # CUDA-event duration over their number is the launch duration the throughput is made of.  The
    # events the library puts around every 64th launch give the duration of a launch taken alone
    # (no overlap with its neighbours' ends, plus the events themselves): reported beside it.
    launch_us = ms_total * 1e3 / (K * layers)  # (ms_total is per block of K steps)
    achieved = algo / (launch_us * 1e-6) / 1e9
    peak, peak_kind = measured_peak_gbs()
    launches = R * K * layers  # one launch per layer-step: the append rides in the attention kernel
    for row in tabs:
        for tb in row:
            lib.qvx_tables_free(tb)

    # ---- e2e: the host-memory call, pinned buffers, copies timed --------------------------------
    qh = torch.empty((s, heads, d), pin_memory=True).normal_(0, scale)
    kh = torch.empty((s, kv_out), pin_memory=True).normal_(0, scale)
    vh = torch.empty((s, kv_out), pin_memory=True).normal_(0, scale)
    oh = [torch.empty((s, heads, d), pin_memory=True) for _ in range(layers)]
    h2d = d2h = 0

    # raw addresses once: the buffers live for the whole run
    p_q, p_k, p_v, p_ta, p_geo = ptr(qh), ptr(kh), ptr(vh), ptr(table_at), C.byref(geo)
    p_blocks, p_out = [ptr(b) for b in layer_blocks], [ptr(o) for o in oh]
    # consecutive ops serve different layers (disjoint blocks): queued together they may overlap each other's ends
    host_variant = qd.ATTN_AUTO | (qd.ATTN_POOL_SETTLED if layers >= 2 else 0)

    def step_host(t: int, pipelined: bool):
        nonlocal h2d, d2h
        pos = (lengths + t).astype(np.uint32)
        p_pos = ptr(pos)
        call = lib.qvx_paged_attention_host_async if pipelined else lib.qvx_paged_attention_host
        for l in range(layers):
            rc = call(dev.h, pool.handle, p_geo, heads, s, p_q, p_k, p_v, p_pos, p_blocks[l], blocks_per_layer, p_ta, None, None, 0,
                      p_out[l], host_variant if pipelined else qd.ATTN_AUTO)
            if rc:
                dev.check(rc)
        if pipelined:
            dev.wait()
        h2d = layers * (qh.numel() * 4 + kh.numel() * 8 + pos.nbytes + table_at.nbytes + layer_blocks[0].nbytes)
        d2h = layers * oh[0].numel() * 4

    def time_host(first: int, pipelined: bool):
        for t in range(first, first + We):
            step_host(t, pipelined)
        barrier()
        each, t0 = [], time.perf_counter()
        for t in range(first + We, first + We + Ke):
            step_host(t, pipelined)
            each.append(time.perf_counter())
        torch.cuda.synchronize()
        el = torch.tensor([time.perf_counter() - t0], device="cuda")
        if dist is not None:
            dist.all_reduce(el, op=dist.ReduceOp.MAX)
        each = [round(1e3 * (b - a), 3) for a, b in zip([t0] + each[:-1], each)]
        return world * s * Ke / float(el.item()), each

    # Both variants step over the same positions (the second rewrites the rows the first wrote).
    e2e_pipelined, each_pipelined = time_host(W + K, True)
    x0 = dev.transfers()
    e2e_value, each_ms = time_host(W + K, False)
    x1 = dev.transfers()
    ops = max(1, x1.submissions - x0.submissions)
    if dist is not None:   # every rank's answer, in rank order
        every = [None] * world
        dist.all_gather_object(every, host_cores)
        host_cores = every
    host_us = {"submit_us_per_op": (x1.submit_ns - x0.submit_ns) / ops / 1e3, "wait_us_per_op": (x1.wait_ns - x0.wait_ns) / ops / 1e3,
               "what": "host time inside qvx_paged_attention_host per layer: queueing the copies and kernels, then waiting for the stream",
               "cores": host_cores}
    checksum = float(sum(float(o[0, 0, 0]) for o in oh))
    assert np.isfinite(checksum)

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms_total / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": config_of(shape, layers),
        "timed_region": {"blocks_of_k_steps": R, "seconds": ms_total * R / 1e3, "pool_gib": pool_blocks * bb / 2**30,
                         "kv_mib_per_launch": algo / 2**20,
                         "value_excludes": "qvx_tables_create (work lists built and uploaded for every step before the clock "
                                           "starts); e2e pays for it in every op"},
        "roofline": {"bound": "hbm", "kernel": "attn_stream_kernel (paged decode attention)", "achieved": achieved, "peak": peak,
                     "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak, "frac_of_8000": achieved / 8000.0,
                     "traffic": algo * DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE, "algorithmic_bytes_per_launch": algo,
                     "launch_us": launch_us, "launches": int(launches),
                     "launch_alone_us": attn_ns / max(attn_launches, 1) / 1e3, "launches_timed_alone": int(attn_launches),
                     "burst": {"launch_us": pilot_ms * 1e3 / (K * layers), "frac": algo / (pilot_ms * 1e-3 / (K * layers)) / 1e9 / peak,
                               "frac_of_8000": algo / (pilot_ms * 1e-3 / (K * layers)) / 1e9 / 8000.0,
                               "what": "the first block of K steps after the warm-up (this rank), tens of milliseconds: the device has "
                                       "not reached its power cap yet; the figures above are the sustained ones"},
                     "kernels_us_per_launch": {k: (v[1] / v[0] / 1e3 if v[0] else 0.0) for k, v in kt.items() if v[0]}},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                "call": "qvx_paged_attention_host x layers per step: synchronous, one op per layer, as DiscreteDevice::routed_moe",
                "d2h_how": "the outputs' host arrays are page-locked: the attention kernel stores into them over the bus while it runs (no copy out)",
                "ms_each_step": each_ms, "host": host_us,
                "pipelined": {"value": e2e_pipelined, "call": "qvx_paged_attention_host_async x layers + qvx_wait per step",
                              "ms_each_step": each_pipelined}},
        "parity_sample": parity,
        "gpu_launches": int(launches),
        "clocks": clocks,
    }
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = CpuSample(shape, lengths, W + K, os.cpu_count() or 1, SEED)
        sec, text = cpu.run(W + K, target_s=12.0)
        sec1, text1 = cpu.run_one_thread(W + K, target_s=3.0)
        line["cpu_baseline"] = {"value": 1.0 / (layers * sec), "unit": UNIT, "cores": os.cpu_count() or 1, "kind": "port", "sample": text,
                                "one_thread": {"value": 1.0 / (layers * sec1), "unit": UNIT, "cores": 1, "sample": text1,
                                               "what": "the same restatement in the device simulation's order, single-threaded"}}
    else:
        line["cpu_baseline"] = None
    pool.free()
    dev.close()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
def run_c5(args, rank: int, local_rank: int, world: int) -> None:
    """The head-sharded configuration: 64 query / 8 KV heads of 128 divided over the ranks by KV head (each
    rank's pool holds its own heads only; block tables replicated), batch 256, contexts U[1024, 16384], one
    layer.  A step = append + attention on every rank, each writing into its slot of the gather buffer, then
    qvx_allgather_heads (ncclAllGather over NVLink + transpose): every rank ends with [token][head][d].
    Afterwards rank 0 recomputes a few sequences with all eight KV heads on its own GPU and compares the
    gathered rows of the last step bit for bit."""
    import torch

    from qubivex_b200 import device as qd
    from qubivex_b200 import sharding
    from qubivex_b200.device import ptr

    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    sampler = ClockSampler(local_rank)
    sampler.start()
    dev = qd.CudaDevice(local_rank, timing=4)
    lib = dev.lib
    shape = wl.C5
    s, d, B = shape.batch, shape.head_dim, shape.block_tokens
    if shape.kv_heads % world:
        raise SystemExit(f"{shape.kv_heads} KV heads do not divide over {world} ranks")
    sh = sharding.head_shard(shape.heads, shape.kv_heads, d, rank, world)
    kvl, hl, group = sh.kv_heads, sh.heads, shape.heads // shape.kv_heads
    W, K = args.warmup, args.steps
    scale = wl.value_scale(shape)
    lengths = wl.contexts(shape, SEED)
    nb_seq = (lengths + W + K + B - 1) // B
    n_blocks = int(nb_seq.sum())
    perm = wl.permutation(n_blocks, SEED)                   # the tables are the same on every rank
    table_at = np.zeros(s, dtype=np.uint32)
    table_at[1:] = np.cumsum(nb_seq)[:-1]
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    gen = torch.Generator(device="cuda")

    def seeded(*key):
        gen.manual_seed(hash((SEED,) + key) & 0x7FFFFFFFFFFFFFFF)
        return gen

    def context_rows(g: int, t: int) -> "torch.Tensor":
        """[position][K row | V row] of KV head g of sequence t: what the prefill leaves in the pool."""
        return torch.randn((int(lengths[t]), 2, d), device="cuda", generator=seeded(1, g, t)) * scale

    def step_inputs(t: int, g: int):
        """q [s][group][d], k_new [s][d], v_new [s][d] of KV head g at step t."""
        x = torch.randn((s, group + 2, d), device="cuda", generator=seeded(2, t, g)) * scale
        return x[:, :group], x[:, group], x[:, group + 1]

    def fill(pool_ptr, geo, pool_blocks, heads_of, seqs, blocks_of, rows_extra=None):
        """Prefill through the sync path: the context rows of the KV heads `heads_of` of sequences `seqs`."""
        for j, t in enumerate(seqs):
            n = int(lengths[t])
            rows = torch.stack([context_rows(g, t) for g in heads_of], dim=2)          # [n][2][heads][d]
            rows = rows.reshape(n, 2 * len(heads_of) * d).contiguous()
            p = np.arange(n)
            to = (blocks_of(j)[p // B].astype(np.int64) * B + p % B).astype(np.uint32)
            d_to = torch.from_numpy(to.view(np.int32)).cuda()
            dev.check(lib.qvx_kv_sync(dev.h, C.byref(geo), pool_ptr, pool_blocks, ptr(rows), ptr(d_to), n, stream))
        torch.cuda.synchronize()

    geo = qd.geometry(B, kvl, d, qd.BF16, qd.LAYOUT_NATIVE)
    bb = qd.block_bytes(geo)
    pool = dev.alloc(n_blocks * bb)
    my_heads = list(range(sh.kv0, sh.kv0 + kvl))
    fill(C.c_void_p(pool.ptr), geo, n_blocks, my_heads, range(s), lambda t: perm[int(table_at[t]):int(table_at[t]) + int(nb_seq[t])])

    def local_inputs(t: int):
        parts = [step_inputs(t, g) for g in my_heads]
        return (torch.cat([p[0] for p in parts], dim=1).contiguous(), torch.cat([p[1] for p in parts], dim=1).contiguous(),
                torch.cat([p[2] for p in parts], dim=1).contiguous())

    inputs = [local_inputs(t) for t in range(W + K)]
    tabs = []
    for t in range(W + K):
        pos = (lengths + t).astype(np.uint32)
        h = C.c_void_p()
        dev.check(lib.qvx_tables_create(dev.h, C.byref(geo), n_blocks, hl, s, ptr(pos), ptr(perm), n_blocks, ptr(table_at), C.byref(h)))
        tabs.append(h)
    uid = [sharding.comm_unique_id() if (rank == 0 and world > 1) else None]
    if dist is not None:
        dist.broadcast_object_list(uid, src=0)
    gather = sharding.HeadGather(dev, world, rank, uid[0], max_tokens=s, heads_local=hl, head_dim=d)
    # The exchange over peer memory where the GPUs reach each other's memory (stores and flags over NVLink, no NCCL call
    # per step); a second communicator stays on NCCL so that both are timed.
    gather_nccl, peer_note = None, "one GPU: nothing to exchange"
    if dist is not None:
        peer_note = "ncclAllGather (in place) + transpose"
        if args.gather == "peer":
            try:
                handles = [None] * world
                dist.all_gather_object(handles, gather.peer_handle())
                gather.peer_open(handles)
                peer_note = "peer memory: each rank stores its rows into every rank's buffer over NVLink, flags, bounded wait, copy out"
            except Exception as e:  # noqa: BLE001 -- no peer access between these devices: NCCL serves
                peer_note += f" (peer memory not available: {e})"
            ok = torch.tensor([1 if gather.over_peer_memory else 0], device="cuda")
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if not int(ok.item()) and gather.over_peer_memory:
                raise SystemExit("peer memory opened on some ranks only")
        if gather.over_peer_memory:
            uid2 = [sharding.comm_unique_id() if rank == 0 else None]
            dist.broadcast_object_list(uid2, src=0)
            gather_nccl = sharding.HeadGather(dev, world, rank, uid2[0], max_tokens=s, heads_local=hl, head_dim=d)
    slot = C.c_void_p(gather.send_slot(s))
    full = torch.empty((s, shape.heads, d), device="cuda")
    pool_p = C.c_void_p(pool.ptr)

    def step(t: int):
        qt, kt, vt = inputs[t]
        dev.check(lib.qvx_kv_append_attn_decode(dev.h, tabs[t], pool_p, ptr(kt), ptr(vt), ptr(qt), slot, qd.ATTN_AUTO, stream))
        gather.all_gather(ptr(full), s, stream)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    for t in range(W):
        step(t)
    barrier()
    dev.reset_kernel_times()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_load0 = time.perf_counter()
    e0.record()
    for t in range(W, W + K):
        step(t)
    e1.record()
    barrier()
    clocks = sampler.stop(t_load0, time.perf_counter())
    ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    if dist is not None:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_total = float(ms.item())
    kt_ = dev.kernel_times()
    last_full = full.clone()
    # the exchange alone: the last step's gather again, bracketed by events (the slot still holds the rank's outputs)
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    g0.record()
    for _ in range(8):
        gather.all_gather(ptr(full), s, stream)
    g1.record()
    barrier()
    gather_us = torch.tensor([g0.elapsed_time(g1) * 1e3 / 8], device="cuda")
    if dist is not None:
        dist.all_reduce(gather_us, op=dist.ReduceOp.MAX)
    nccl_us = None
    if gather_nccl is not None:                     # the same exchange through NCCL, for comparison (its slot's contents do not matter)
        for _ in range(3):
            gather_nccl.all_gather(ptr(full), s, stream)
        barrier()
        g0.record()
        for _ in range(8):
            gather_nccl.all_gather(ptr(full), s, stream)
        g1.record()
        barrier()
        nccl_us = torch.tensor([g0.elapsed_time(g1) * 1e3 / 8], device="cuda")
        dist.all_reduce(nccl_us, op=dist.ReduceOp.MAX)
        nccl_us = float(nccl_us.item())
        gather.all_gather(ptr(full), s, stream)     # (the result buffer again holds the last step's rows)
        torch.cuda.synchronize()

    # ---- e2e: the step's q, k_new, v_new from pinned host memory, the gathered result back to the host -----------
    hq, hk, hv = (torch.empty_like(x, device="cpu").pin_memory() for x in inputs[W + K - 1])
    for hbuf, x in zip((hq, hk, hv), inputs[W + K - 1]):
        hbuf.copy_(x)
    dq, dk, dv = (torch.empty_like(x) for x in inputs[W + K - 1])
    hfull = torch.empty((s, shape.heads, d), pin_memory=True)
    t_e2e = min(W + K - 1, W + 7)

    def step_host():
        dq.copy_(hq, non_blocking=True); dk.copy_(hk, non_blocking=True); dv.copy_(hv, non_blocking=True)
        dev.check(lib.qvx_kv_append_attn_decode(dev.h, tabs[W + K - 1], pool_p, ptr(dk), ptr(dv), ptr(dq), slot, qd.ATTN_AUTO, stream))
        gather.all_gather(ptr(full), s, stream)
        hfull.copy_(full, non_blocking=True)
        torch.cuda.synchronize()

    for _ in range(3):
        step_host()
    barrier()
    t0 = time.perf_counter()
    n_e2e = max(4, min(K, 16))
    for _ in range(n_e2e):
        step_host()
    el = torch.tensor([time.perf_counter() - t0], device="cuda")
    if dist is not None:
        dist.all_reduce(el, op=dist.ReduceOp.MAX)
    e2e_value = s * n_e2e / float(el.item())

    # ---- the check against one GPU: rank 0 recomputes a few sequences with all eight KV heads ------------------
    check = None
    if rank == 0:
        sample = sorted({int(np.argmin(lengths)), int(np.argsort(lengths)[s // 2]), int(np.argmax(lengths))})
        geo1 = qd.geometry(B, shape.kv_heads, d, qd.BF16, qd.LAYOUT_NATIVE)
        nb1 = nb_seq[sample]
        ta1 = np.zeros(len(sample), dtype=np.uint32)
        ta1[1:] = np.cumsum(nb1)[:-1]
        blocks1 = np.arange(int(nb1.sum()), dtype=np.uint32)
        pool1 = dev.alloc(int(nb1.sum()) * qd.block_bytes(geo1))
        all_heads = list(range(shape.kv_heads))
        fill(C.c_void_p(pool1.ptr), geo1, int(nb1.sum()), all_heads, sample, lambda j: blocks1[int(ta1[j]):int(ta1[j]) + int(nb1[j])])
        out1 = torch.empty((len(sample), shape.heads, d), device="cuda")
        idx = torch.tensor(sample, device="cuda")
        for t in range(W + K):                                   # every step's rows land as they did in the run; the last one's outputs count
            parts = [step_inputs(t, g) for g in all_heads]
            q1 = torch.cat([p[0][idx] for p in parts], dim=1).contiguous()
            k1 = torch.cat([p[1][idx] for p in parts], dim=1).contiguous()
            v1 = torch.cat([p[2][idx] for p in parts], dim=1).contiguous()
            pos1 = (lengths[sample] + t).astype(np.uint32)
            h = C.c_void_p()
            dev.check(lib.qvx_tables_create(dev.h, C.byref(geo1), int(nb1.sum()), shape.heads, len(sample), ptr(pos1), ptr(blocks1),
                                            len(blocks1), ptr(ta1), C.byref(h)))
            dev.check(lib.qvx_kv_append_attn_decode(dev.h, h, C.c_void_p(pool1.ptr), ptr(k1), ptr(v1), ptr(q1), ptr(out1), qd.ATTN_AUTO, stream))
            torch.cuda.synchronize()
            lib.qvx_tables_free(h)
        got = last_full[idx]
        same = bool(torch.equal(got.view(torch.int32), out1.view(torch.int32)))
        check = {"sequences": sample, "contexts": [int(lengths[i]) + W + K for i in sample], "bit_identical": same,
                 "max_abs_diff": float((got - out1).abs().max()), "what": "rank 0's gathered [token][head][d] rows of the last step against "
                 "the same steps run with all 8 KV heads on one GPU"}
        pool1.free()

    attn_launches, attn_ns = kt_["attn"]
    algo_rank = float(np.mean([wl.algorithmic_bytes(dataclasses.replace(shape, heads=hl, kv_heads=kvl), lengths + t + 1)
                               for t in range(W, W + K)]))
    peak, peak_kind = measured_peak_gbs()
    attn_us = attn_ns / max(attn_launches, 1) / 1e3
    value = s * K / (ms_total / 1e3)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_total / K,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": shape.name, "layers": 1, "batch": s, "heads": shape.heads, "kv_heads": shape.kv_heads, "head_dim": d,
                   "block_tokens": B, "context": [shape.ctx_lo, shape.ctx_hi],
                   "partition": f"by KV head: {kvl} KV head(s) and {hl} query heads per GPU; one exchange of the outputs per step (the gather object says which)",
                   "l2": f"each launch reads {algo_rank / 2**20:.0f} MiB of KV per GPU, once: no flush between iterations"},
        "roofline": {"bound": "hbm", "kernel": "attn_stream_kernel (paged decode attention), per GPU", "achieved": algo_rank / (attn_us * 1e-6) / 1e9,
                     "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": algo_rank / (attn_us * 1e-6) / 1e9 / peak,
                     "frac_of_8000": algo_rank / (attn_us * 1e-6) / 1e9 / 8000.0, "traffic": None,
                     "algorithmic_bytes_per_launch": algo_rank, "launch_us": attn_us, "launches_timed": int(attn_launches),
                     "how": "CUDA events around every 4th attention launch of the timed region (slowest rank not taken: this rank's)"},
        "gather": {"us_per_step": float(gather_us.item()), "bytes_gathered_per_gpu": s * shape.heads * d * 4, "path": peer_note,
                   "nccl_us_per_step": nccl_us, "what": "8 exchanges in a row bracketed by CUDA events, slowest rank"},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(world * (hq.numel() + hk.numel() + hv.numel()) * 4),
                "d2h_bytes_per_step": int(world * hfull.numel() * 4),
                "call": "per rank and step: q, k_new, v_new from pinned host memory, qvx_kv_append_attn_decode into the gather slot, "
                        "qvx_allgather_heads, the gathered result back to pinned host memory, synchronize"},
        "check_vs_one_gpu": check,
        "gpu_launches": int(2 * K),
        "clocks": clocks,
        "cpu_baseline": None,
    }
    for h in tabs:
        lib.qvx_tables_free(h)
    gather.close()
    if gather_nccl is not None:
        gather_nccl.close()
    pool.free()
    dev.close()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--config", choices=["c2", "c5"], default="c2",
                    help="c2: the MoE-decoder configuration the metric is quoted on, partitioned by sequence (default); "
                         "c5: the head-sharded configuration, one all-gather per step")
    ap.add_argument("--gather", choices=["peer", "nccl"], default="peer",
                    help="c5: the outputs' exchange over peer memory where the GPUs allow it (default), or through NCCL only")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration's 48 (debugging only)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--min-seconds", type=float, default=1.0, help="the K steps are repeated until the timed region lasts this long")
    args = ap.parse_args()
    rank, local_rank, world = env_int("RANK", 0), env_int("LOCAL_RANK", 0), env_int("WORLD_SIZE", 1)
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        if world != args.gpus and world > 1:
            raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
        (run_c5 if args.config == "c5" else run_ours)(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
