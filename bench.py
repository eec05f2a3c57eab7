#!/usr/bin/env python
"""Benchmark of the attention/encoder hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload prefill|decode|encoder|layernorm] [--impl ours|reference]

One JSON line on stdout (rank 0). The headline workload is the long-sequence prefill attention of the baseline's
config 4 (batch 4 x 16 heads, head_dim 128, bf16, seq 8192, no mask), run as the baseline names it: the ONE
configuration is sharded by head over the N ranks (16/N heads each, strong scaling) and every rank ends the step
holding the whole attention output [4, 8192, 16 x 128] (the all-gather at the attention-output boundary). At N > 1 the
step is timed twice, with the delivery done by an NCCL all-gather after the kernel and by the attention kernel itself
storing its tiles into every rank's buffer over peer memory (vkc_attn_prefill_fanout + a bounded flag wait); `value`
is the better one, both are in `extra.strong`. `value` is measured with inputs resident in HBM; `e2e` is the same
metric through the C-ABI with pinned HOST buffers (vkc_upload -> kernel -> vkc_download of every step inside the timed
region, consecutive steps pipelined over three streams so that the copies overlap the kernel). `extra` carries the
other parts of the baseline's composite metric (decode GB/s, encoder tok/s, the rest of the prefill sweep), each with
its own roofline, a sustained (>= 2 s) run of the headline kernel, the Session::run wall through the C++ plug-in, and,
at N > 1, the weak-scaling figures and the one-sequence encoder legs with their deviation from the single-GPU result.

Inputs are synthetic (seeded N(0,1)); they stand in for the shapes the baseline names. Between timed steps the
kernels cycle through several input sets so that every step reads data that is not L2 resident.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

L2_BYTES = 126 * 1024 * 1024
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# DRAM traffic per unit (dram__bytes_read.sum + dram__bytes_write.sum) from one ncu capture per kernel:
#   prefill  : 111.72 MB for 4 x 16 x 2048 (batch, head, query row) units; K/V re-reads are served by L2, so DRAM traffic
#              grows with the number of row units;
#   decode   : 1.021 x the algorithmic bytes of the launch;
#   layernorm: 1.0 x (the capture moved the algorithmic bytes; hit rate 3.6 %).
NCU_PREFILL_DRAM_BYTES_PER_ROW_UNIT = 852.4
NCU_DECODE_DRAM_OVER_ALGORITHMIC = 1.021

PREFILL = dict(B=4, H=16, S=8192, D=128, causal=False, dtype="bf16", seed=1005)
DECODE = dict(B=32, Hq=32, Hkv=8, L=8192, D=128, seed=1005)
ENCODER = dict(B=8, T=197, d=768, H=12, dmlp=3072, seed=1002)
STACK = dict(B=1, T=2738, d=1024, H=16, dmlp=4096, layers=24, seed=1003)  # config 3
LAYERNORM = dict(rows=131072, norm=1024, seed=1003)  # config 3's width; enough rows that the pass streams from HBM


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        d["_source"] = "measured"
        return d
    d = dict(FALLBACK_PEAKS)
    d["_source"] = "fallback"
    return d


class ClockSampler:
    """Samples SM clock, power and the clock-event reasons of one GPU in a thread while the benchmark runs (read-only NVML
    queries every few milliseconds; `nvidia-smi` every 100 ms where the NVML binding is missing). Every sample carries a
    host time stamp, so a timed region asks for the samples that fell inside it."""
    REASONS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20), ("sw_power_cap", 0x4))
    Q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index, uuid=None):
        self.rows, self.index, self.uuid = [], index, uuid  # rows: (t, sm_mhz, power_w, reasons bitmask)
        self.max_mhz, self.stop_flag, self.thread, self.proc, self.how = None, False, None, None, None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            h = None
            if self.uuid:
                for u in (self.uuid, self.uuid.encode()):
                    try:
                        h = pynvml.nvmlDeviceGetHandleByUUID(u)
                        break
                    except Exception:  # noqa: BLE001
                        h = None
            if h is None:
                h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            self.how = "nvml"

            def loop():
                while not self.stop_flag:
                    try:
                        mhz = pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)
                        mask = pynvml.nvmlDeviceGetCurrentClocksEventReasons(h)
                        try:
                            watts = pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0
                        except Exception:  # noqa: BLE001
                            watts = None
                        self.rows.append((time.perf_counter(), float(mhz), watts, int(mask)))
                    except Exception:  # noqa: BLE001
                        pass
                    time.sleep(0.004)
            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
            return
        except Exception:  # noqa: BLE001
            self.how = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.how = "nvidia-smi"

            def read():
                for line in self.proc.stdout:
                    r = [c.strip() for c in line.split(",")]
                    try:
                        mask = 0
                        for (name, bit), v in zip(self.REASONS, r[3:7]):
                            if v.lower().startswith("active"):
                                mask |= bit
                        self.max_mhz = float(r[1])
                        self.rows.append((time.perf_counter(), float(r[0]), float(r[2]), mask))
                    except (ValueError, IndexError):
                        continue
            self.thread = threading.Thread(target=read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def stop(self):
        self.stop_flag = True
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        if self.thread:
            self.thread.join(timeout=2)

    def window(self, t0, t1):
        """Summary of the samples taken between two host times (perf_counter)."""
        if self.how is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["clock sampling unavailable"], "samples": 0}
        rows = [r for r in self.rows if t0 <= r[0] <= t1]
        if not rows and self.rows:  # a region shorter than the sampling period: take the nearest sample
            rows = [min(self.rows, key=lambda r: abs(r[0] - 0.5 * (t0 + t1)))]
        mask = 0
        for r in rows:
            mask |= r[3]
        watts = [r[2] for r in rows if r[2] is not None]
        return {"sm_mhz": float(np.median([r[1] for r in rows])) if rows else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(n for n, bit in self.REASONS if mask & bit), "samples": len(rows),
                "power_w_max": max(watts) if watts else None, "source": self.how}


# ---------------------------------------------------------------------------------------------------------------
def dist_setup(n):
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(0)
    return rank, world, local


def barrier(world):
    import torch
    import torch.distributed as dist
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(x, world):
    import torch
    import torch.distributed as dist
    if world == 1:
        return float(x)
    t = torch.tensor([float(x)], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(x, world):
    import torch
    import torch.distributed as dist
    if world == 1:
        return float(x)
    t = torch.tensor([float(x)], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


LAST_WINDOW = [0.0, 0.0]  # host times (perf_counter) bracketing the most recent timed loop


def timed_loop(fn, steps, warmup, world):
    """W untimed steps, then exactly K steps between barrier+synchronize; per-step CUDA events on the launching
    stream. Returns (total_ms as max over ranks, mean per-launch ms on this rank)."""
    import torch
    for i in range(warmup):
        fn(i)
    barrier(world)
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    LAST_WINDOW[0] = time.perf_counter()
    evs[0].record()
    for i in range(steps):
        fn(warmup + i)
        evs[i + 1].record()
    barrier(world)
    LAST_WINDOW[1] = time.perf_counter()
    total = evs[0].elapsed_time(evs[-1])
    per = [evs[i].elapsed_time(evs[i + 1]) for i in range(steps)]
    return max_over_ranks(total, world), float(np.mean(per))


def n_sets_for(bytes_per_step):
    return max(2, int(np.ceil(2.0 * L2_BYTES / max(bytes_per_step, 1))) + 1)


def tensor_roofline(flops, ms, pk, traffic=None, kernel=None, **more):
    a = flops / (ms * 1e-3) / 1e12
    r = {"bound": "tensor", "achieved": a, "peak": pk["bf16_tflops"], "unit": "TFLOP/s", "frac": a / pk["bf16_tflops"], "traffic": traffic,
         "peak_source": "%s 16-bit dense burst (cuBLAS)" % pk["_source"]}
    if kernel:
        r["kernel"] = kernel
    r.update(more)
    return r


def hbm_roofline(nbytes, ms, pk, traffic=None, kernel=None, **more):
    a = nbytes / (ms * 1e-3) / 1e9
    r = {"bound": "hbm", "achieved": a, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": a / pk["hbm_gbs"], "traffic": traffic,
         "peak_source": "%s copy bandwidth" % pk["_source"]}
    if kernel:
        r["kernel"] = kernel
    r.update(more)
    return r


# ---------------------------------------------------------------------------------------------------------------
def prefill_flops(cfg, heads):
    B, S, D = cfg["B"], cfg["S"], cfg["D"]
    return (2 * B * heads * S * (S + 1) * D) if cfg["causal"] else (4 * B * heads * S * S * D)


def bench_prefill(ctx, cfg, steps, warmup, rank, world, e2e_steps=0, heads_per_rank=None, sustained_s=0.0, sampler=None):
    """The fused attention kernel over `heads_per_rank` heads of the configuration on every rank (default: all of them),
    no delivery of the output. Returns times, the per-launch figure and, on request, the end-to-end and sustained legs."""
    import torch
    B, H, S, D = cfg["B"], cfg["H"], cfg["S"], cfg["D"]
    Hl = heads_per_rank or H
    dt = torch.bfloat16
    g = torch.Generator(device="cuda").manual_seed(cfg["seed"] + rank)
    bytes_step = 4 * B * Hl * S * D * 2
    ns = min(n_sets_for(bytes_step), 6)
    sets = []
    for _ in range(ns):
        q, k, v = (torch.randn(B, Hl, S, D, generator=g, device="cuda", dtype=torch.float32).to(dt) for _ in range(3))
        sets.append((q, k, v, torch.empty_like(q)))
    scale = 1.0 / float(np.sqrt(D))

    def step(i):
        q, k, v, o = sets[i % ns]
        ctx.attn_prefill(q, k, v, o, scale, causal=cfg["causal"])

    n0 = ctx.launch_count()
    total_ms, per_launch_ms = timed_loop(step, steps, warmup, world)
    launches = ctx.launch_count() - n0 - warmup
    window = tuple(LAST_WINDOW)
    ctx.sync()
    flops_rank = prefill_flops(cfg, Hl)
    res = dict(total_ms=total_ms, per_launch_ms=per_launch_ms, flops_step_rank=flops_rank, launches=launches, bytes_step_rank=bytes_step, n_sets=ns,
               window=window, heads_per_rank=Hl)

    if sustained_s > 0:
        # the same launch back to back for at least `sustained_s` seconds between two events: the figure under the power cap
        n_est = max(steps, int(np.ceil(sustained_s * 1e3 / max(per_launch_ms, 1e-3) * 1.15)))
        barrier(world)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        for i in range(n_est):
            step(i)
        e1.record()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        ms = e0.elapsed_time(e1)
        ctx.sync()
        clk = sampler.window(t0 + 0.1 * (t1 - t0), t1) if sampler else None  # skip the ramp at the start of the window
        res["sustained"] = dict(tflops=flops_rank * n_est / (ms * 1e-3) / 1e12, seconds=ms * 1e-3, launches=n_est,
                                sm_mhz_median=clk["sm_mhz"] if clk else None, clock_samples=clk["samples"] if clk else 0,
                                reasons=clk["reasons"] if clk else None, power_w_max=clk.get("power_w_max") if clk else None)

    # end to end through the C-ABI with host buffers
    if e2e_steps > 0:
        q, k, v, o = sets[0]
        hq, hk, hv = (torch.empty(t.shape, dtype=dt).pin_memory() for t in (q, k, v))
        ho = torch.empty(o.shape, dtype=dt).pin_memory()
        hq.copy_(q)
        hk.copy_(k)
        hv.copy_(v)

        # Every step uploads its Q, K, V from pinned host memory, runs the kernel and downloads O, all through the C-ABI.
        # Steps are pipelined over three streams and two device buffer sets, as a serving loop would do: the upload of
        # step i+1 and the download of step i-1 run under the kernel of step i (PCIe is full duplex), so the steady state
        # costs max(upload, kernel, download) per step instead of their sum. Every copy of every step is inside the timed
        # region. With several ranks each rank moves its own heads; the host holds the whole output once all have downloaded.
        s_up, s_run, s_down = (torch.cuda.Stream() for _ in range(3))
        bufs = [sets[0], sets[1 % ns]]
        up_done = [torch.cuda.Event() for _ in range(2)]
        run_done = [torch.cuda.Event() for _ in range(2)]
        down_done = [torch.cuda.Event() for _ in range(2)]

        def e2e(i):
            b = i % 2
            bq, bk, bv, bo = bufs[b]
            if i >= 2:
                s_up.wait_event(run_done[b])       # the kernel two steps back has read this buffer set
                s_run.wait_event(down_done[b])     # and its output has left the device
            for t, h in ((bq, hq), (bk, hk), (bv, hv)):
                ctx.upload_ptr(t, h.data_ptr(), 2, stream=s_up.cuda_stream)
            up_done[b].record(s_up)
            s_run.wait_event(up_done[b])
            ctx.attn_prefill(bq, bk, bv, bo, scale, causal=cfg["causal"], stream=s_run.cuda_stream)
            run_done[b].record(s_run)
            s_down.wait_event(run_done[b])
            ctx.download_ptr(ho.data_ptr(), 2, bo, stream=s_down.cuda_stream)
            down_done[b].record(s_down)

        def e2e_timed(n_steps, n_warm):
            cur = torch.cuda.current_stream()
            for i in range(n_warm):
                e2e(i)
            for st in (s_up, s_run, s_down):
                cur.wait_stream(st)
            barrier(world)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(cur)
            for st in (s_up, s_run, s_down):
                st.wait_event(e0)
            for i in range(n_steps):
                e2e(n_warm + i)
            for st in (s_up, s_run, s_down):
                cur.wait_stream(st)
            e1.record(cur)
            barrier(world)
            return max_over_ranks(e0.elapsed_time(e1), world)

        t_ms = e2e_timed(e2e_steps, 2)
        res["e2e_ms_per_step"] = t_ms / e2e_steps
        res["e2e_steps"] = e2e_steps
        res["h2d"] = 3 * q.numel() * 2 * world
        res["d2h"] = o.numel() * 2 * world
    return res


def bench_prefill_delivered(ctx, cfg, steps, warmup, rank, world):
    """Strong scaling of the ONE named configuration: rank r computes heads [r*H/N, (r+1)*H/N) of every batch element and
    the step ends when every rank holds the whole output. Timed twice: (a) kernel, then one NCCL all-gather; (b) the
    kernel stores each output row into every rank's [B, S, H*D] buffer over peer memory and raises a flag, the step ends
    with a bounded device-side wait for all ranks' flags. Returns both and a correctness figure for (b) against (a)."""
    import torch
    import torch.distributed as dist
    from vknn_b200.sharding import PeerGather
    B, H, S, D = cfg["B"], cfg["H"], cfg["S"], cfg["D"]
    Hl = H // world
    dt = torch.bfloat16
    g = torch.Generator(device="cuda").manual_seed(cfg["seed"] + rank)
    bytes_step = 3 * B * Hl * S * D * 2
    ns = min(n_sets_for(bytes_step), 6)
    sets = [tuple(torch.randn(B, Hl, S, D, generator=g, device="cuda", dtype=torch.float32).to(dt) for _ in range(3)) for _ in range(ns)]
    scale = 1.0 / float(np.sqrt(D))
    out = {}

    # (a) NCCL: the gathered buffer is rank-major [N, B, Hl, S, D]; a rank writes its slice and gathers in place
    full = torch.empty(world, B, Hl, S, D, dtype=dt, device="cuda")

    def step_nccl(i):
        q, k, v = sets[i % ns]
        ctx.attn_prefill(q, k, v, full[rank], scale, causal=cfg["causal"])
        dist.all_gather_into_tensor(full.view(world, -1), full[rank].view(-1))

    t_ms, _ = timed_loop(step_nccl, steps, warmup, world)
    ctx.sync()
    out["nccl_allgather"] = dict(ms_per_step=t_ms / steps)
    q0, k0, v0 = sets[0]
    step_nccl(0)
    torch.cuda.synchronize()
    want = full.permute(1, 3, 0, 2, 4).reshape(B, S, H * D).clone()  # [N,B,Hl,S,D] -> merged-head [B, S, (N Hl) D]

    # (b) fused: every rank's buffer is the merged-head layout [B*S, H*D] the out-projection would read
    try:
        gather = PeerGather(ctx, B * S, H * D, dt)
        o_strides = (S * H * D, D, H * D)

        def step_fused(i):
            q, k, v = sets[i % ns]
            kb = gather.next_buffer()
            ctx.attn_prefill_fanout(q, k, v, gather.dests(kb, rank * Hl * D), gather.flags(), gather.state, o_strides, scale, causal=cfg["causal"],
                                    mcast=gather.mcast(kb, rank * Hl * D))
            gather.wait()
            return kb

        kb = step_fused(0)
        ctx.sync()
        dist.barrier()
        err = float((gather.buffers[kb].view(B, S, H * D).float() - want.float()).abs().max())
        step_fused(1)  # keep the two buffers alternating in step with the other ranks
        ctx.sync()
        dist.barrier()
        f_ms, _ = timed_loop(step_fused, steps, warmup + (warmup % 2), world)
        ctx.sync()
        out["fused_fanout"] = dict(ms_per_step=f_ms / steps, max_abs_vs_nccl_path=max_over_ranks(err, world),
                                   stores="one multimem store per 16 bytes, replicated by the NVSwitch" if gather.mcast_base else "one peer store per destination")
        dist.barrier()
        gather.close()
    except Exception as e:  # noqa: BLE001 - peer memory unavailable on this box: the NCCL figure stands
        out["fused_fanout"] = dict(unavailable=str(e)[:300])
    del full, want
    return out


def bench_decode(ctx, cfg, steps, warmup, rank, world, strong=False):
    import torch
    B, Hq, Hkv, L, D = cfg["B"], cfg["Hq"], cfg["Hkv"], cfg["L"], cfg["D"]
    if strong:
        # the ONE named batch of 32 sequences, 32/N per rank (same seeded lengths at every N), no collective
        lens_all = np.random.default_rng(cfg["seed"]).integers(1024, L + 1, B).astype(np.int32)
        Bl = B // world
        kv_len = lens_all[rank * Bl:(rank + 1) * Bl].copy()
    else:
        Bl = B  # weak scaling: every rank serves the named configuration's 32 sequences (world x 32 in total)
        kv_len = np.random.default_rng(cfg["seed"] + 1000 * rank).integers(1024, L + 1, B).astype(np.int32)
    g = torch.Generator(device="cuda").manual_seed(cfg["seed"] + rank)
    dt = torch.float16
    bytes_alg = int(2 * Hkv * int(kv_len.sum()) * D * 2 + 2 * Bl * Hq * D * 2)
    ns = min(n_sets_for(bytes_alg), 6 if strong else 4)
    sets = []
    for _ in range(ns):
        k = torch.randn(Bl, Hkv, L, D, generator=g, device="cuda", dtype=dt)
        v = torch.randn(Bl, Hkv, L, D, generator=g, device="cuda", dtype=dt)
        q = torch.randn(Bl, Hq, D, generator=g, device="cuda", dtype=dt)
        sets.append((q, k, v, torch.empty_like(q)))
    lens = torch.from_numpy(kv_len).cuda()
    ws = torch.empty(ctx.attn_decode_workspace_bytes(Bl, Hq, Hkv, L, D), dtype=torch.uint8, device="cuda")
    scale = 1.0 / float(np.sqrt(D))

    def eager(i):
        q, k, v, o = sets[i % ns]
        ctx.attn_decode(q, k, v, o, scale, kv_len=lens, workspace=ws)

    # a decode step is one short launch: replay it from a CUDA graph, as a serving loop would
    for i in range(ns):
        eager(i)
    torch.cuda.synchronize()
    graphs = []
    for i in range(ns):
        g_ = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_):
            eager(i)
        graphs.append(g_)

    def step(i):
        graphs[i % ns].replay()

    total_ms, per_ms = timed_loop(eager if os.environ.get("VKNN_BENCH_EAGER") == "1" else step, steps, warmup, world)
    ctx.sync()
    bytes_all = sum_over_ranks(bytes_alg, world)
    return dict(total_ms=total_ms, per_launch_ms=per_ms, bytes_step_all=bytes_all, bytes_step_rank=bytes_alg, gbs=bytes_all * steps / (total_ms * 1e-3) / 1e9)


NO_TUNE = False


def bench_encoder(ctx, cfg, steps, warmup, rank, world):
    import torch
    from vknn_b200.synthetic import encoder_weights
    from vknn_b200.encoder import EncoderLayer
    B, T, d, H, dm = cfg["B"], cfg["T"], cfg["d"], cfg["H"], cfg["dmlp"]
    Bl = B  # weak scaling: every rank runs the named batch of 8 images (world x 8 in total), weights replicated
    w = encoder_weights(np.random.default_rng(cfg["seed"]), d, dm)
    layer = EncoderLayer(ctx, w, H, dtype=torch.float16)
    g = torch.Generator(device="cuda").manual_seed(cfg["seed"] + rank)
    # the layer's weights (14 MB) are reused every step by design; activations cycle through enough sets to leave L2
    ns = 8
    xs = [torch.randn(Bl, T, d, generator=g, device="cuda", dtype=torch.float32).half() for _ in range(ns)]
    ys = [torch.empty_like(x) for x in xs]

    # the layer is 7 short launches: replay it as a CUDA graph (what the C++ segment does), one graph per input set
    layer.forward(xs[0], out=ys[0])
    if not NO_TUNE:
        layer.tune(xs[0])  # per-shape GEMM configuration by measurement, as the C++ segment does at plan time (Hint::Tuning)
    for i in range(ns):
        layer.forward(xs[i], out=ys[i])
    torch.cuda.synchronize()
    graphs = [layer.capture(xs[i], ys[i]) for i in range(ns)]

    def step(i):
        graphs[i % ns].replay()

    total_ms, per_ms = timed_loop(step, steps, warmup, world)
    ctx.sync()
    tokens_all = B * T * world
    return dict(total_ms=total_ms, per_launch_ms=per_ms, tok_s=tokens_all * steps / (total_ms * 1e-3), flops_step_rank=layer.flops(Bl, T),
                tflops=layer.flops(Bl, T) * world * steps / (total_ms * 1e-3) / 1e12)


def bench_stack(ctx, cfg, steps, warmup, rank, world):
    """Config 3: 24 pre-LN blocks, d=1024, 16 heads, MLP 4096, 2738 tokens, batch 1. Weak scaling runs one sequence
    per rank (graph replay); with more than one rank the same stack is also run head-sharded on ONE shared sequence
    (QKV + attention sharded by head, one NCCL all-gather per layer at the attention output, the rest replicated), and then
    twice more without any collective call: with the attention kernel storing its tiles into every rank's gather buffer
    over peer memory, and with the tokens sharded as well (LayerNorm 1 fans its rows out the same way). Each sharded leg
    reports its largest deviation from the single-GPU forward of the same sequence (max over ranks)."""
    import torch
    from vknn_b200.encoder import EncoderStack
    from vknn_b200.synthetic import encoder_weights
    T, d, H, dm, L = cfg["T"], cfg["d"], cfg["H"], cfg["dmlp"], cfg["layers"]
    rng = np.random.default_rng(cfg["seed"])
    stack = EncoderStack(ctx, [encoder_weights(rng, d, dm) for _ in range(L)], H, dtype=torch.float16)
    g = torch.Generator(device="cuda").manual_seed(cfg["seed"] + rank)
    x = torch.randn(1, T, d, generator=g, device="cuda", dtype=torch.float32).half()
    stack.forward(x)
    if not NO_TUNE:
        stack.tune(x)
    stack.forward(x)
    torch.cuda.synchronize()
    graph, _ = stack.capture(x)
    total_ms, per_ms = timed_loop(lambda i: graph.replay(), steps, warmup, world)
    ctx.sync()
    res = dict(tok_s=T * world * steps / (total_ms * 1e-3), ms_per_forward=total_ms / steps, per_launch_ms=per_ms, flops_step_rank=stack.flops(1, T),
               tflops=stack.flops(1, T) * world * steps / (total_ms * 1e-3) / 1e12)
    if world > 1:
        import torch.distributed as dist
        from vknn_b200.sharding import shard_range
        xs = x.clone()
        dist.broadcast(xs, 0)
        ref = stack.forward(xs).clone()  # the single-GPU answer for the shared sequence (weights are replicated)
        ctx.sync()
        ref_max = float(ref.float().abs().max())  # the residual stream reaches O(10..100) after 24 blocks: one fp16 ulp there is 0.03

        def dev(y, r=None):
            return max_over_ranks(float((y.float() - (ref if r is None else r).float()).abs().max()), world)
        stack.shard_heads(rank, world)
        y = stack.forward_head_sharded(xs)
        ctx.sync()
        err = dev(y)
        t_ms, _ = timed_loop(lambda i: stack.forward_head_sharded(xs), steps, warmup, world)
        ctx.sync()
        res["head_sharded_one_sequence"] = dict(tok_s=T * steps / (t_ms * 1e-3), ms_per_forward=t_ms / steps, max_abs_vs_single_gpu=err, max_abs_of_output=ref_max,
                                                note="strong scaling of a single sequence: QKV+attention sharded by head, all-gather per layer, "
                                                     "out-projection and MLP replicated (about half of the flops do not shard)")
        if world <= 8 and L % 2 == 0:
            try:
                # the same without a collective: the attention kernel stores its tiles into every rank's gather buffer over peer
                # memory and raises a flag; the whole forward is one CUDA graph per rank
                from vknn_b200.sharding import PeerGather
                gather = PeerGather(ctx, T, d, torch.float16)
                y = stack.forward_head_sharded_fused(xs, gather)
                ctx.sync()
                err = dev(y)
                dist.barrier()
                fgraph, _ = stack.capture_head_sharded_fused(xs, gather)
                f_ms, _ = timed_loop(lambda i: fgraph.replay(), steps, warmup, world)
                ctx.sync()
                res["head_sharded_one_sequence_fused"] = dict(tok_s=T * steps / (f_ms * 1e-3), ms_per_forward=f_ms / steps, max_abs_vs_single_gpu=err, max_abs_of_output=ref_max,
                                                              note="attention output fanned out by the attention kernel over peer memory "
                                                                   "(no NCCL call in the forward), graph replay")
                dist.barrier()
                # tokens sharded too (out-projection and MLP on T/world rows per rank): LayerNorm 1 and the attention kernel each
                # fan their output out to every rank, two flag waits per layer, still no collective call and one graph per rank
                gh = PeerGather(ctx, T, d, torch.float16)
                y = stack.forward_token_sharded(xs, gh, gather)
                ctx.sync()
                lo, hi = shard_range(T, rank, world)
                err = dev(y, ref.view(T, d)[lo:hi])
                dist.barrier()
                tgraph, _ = stack.capture_token_sharded(xs, gh, gather)
                t2_ms, _ = timed_loop(lambda i: tgraph.replay(), steps, warmup, world)
                ctx.sync()
                res["token_and_head_sharded_one_sequence"] = dict(tok_s=T * steps / (t2_ms * 1e-3), ms_per_forward=t2_ms / steps, max_abs_vs_single_gpu=err, max_abs_of_output=ref_max,
                                                                  note="every GEMM, LayerNorm and the attention sharded; the two gathers per layer "
                                                                       "are stores of the producing kernels over peer memory; output left sharded by rows")
                dist.barrier()
                gh.close()
                gather.close()
            except Exception as e:  # noqa: BLE001 - peer memory unavailable on this box: keep the rest of the line
                res["peer_memory_legs"] = dict(unavailable=str(e)[:300])
    return res


def bench_layernorm(ctx, cfg, steps, warmup, rank, world):
    import torch
    rows, norm = cfg["rows"], cfg["norm"]
    g = torch.Generator(device="cuda").manual_seed(cfg["seed"] + rank)
    xs = [torch.randn(rows, norm, generator=g, device="cuda", dtype=torch.float32).half() for _ in range(2)]
    ys = [torch.empty_like(x) for x in xs]
    gamma = torch.ones(norm, device="cuda")
    beta = torch.zeros(norm, device="cuda")

    def step(i):
        ctx.layernorm(xs[i % 2], gamma, beta, ys[i % 2], 1e-6)

    total_ms, per_ms = timed_loop(step, steps, warmup, world)
    ctx.sync()
    bytes_rank = rows * norm * 2 * 2 + 8 * norm
    return dict(total_ms=total_ms, per_launch_ms=per_ms, bytes_step_rank=bytes_rank, gbs=bytes_rank * world * steps / (total_ms * 1e-3) / 1e9)


def bench_raster(ctx, steps, warmup, rank, world):
    """The reference's renderer size: 100352 gaussians, one 224 x 224 view (seeded synthetic splats stand in for the
    encoder's outputs). One step = project + depth sort + composite; double (specification-exact) and float arithmetic."""
    import torch
    from vknn_b200.synthetic import splat_scene
    H = W = 224
    n = 100352
    means, covs, colors, opac, w2c, K = splat_scene(1006 + rank, n, H, W)
    dev = [torch.from_numpy(a).cuda() for a in (means, covs, colors, opac)]
    out = {}
    for name, precise in (("f64", True), ("f32", False)):
        total_ms, _ = timed_loop(lambda i: ctx.raster_gaussians(*dev, w2c, K, H, W, near=0.2, precise=precise), steps, warmup, world)
        ctx.sync()
        out["ms_per_view_" + name] = total_ms / steps
    out["workload"] = "3D Gaussian splatting: 100352 gaussians, one 224 x 224 view per rank"
    out["algorithmic_bytes"] = n * 100 + H * W * 16
    return out


def plugin_e2e():
    """Session::run wall (host fp32 in, host fp32 out, boundary copies and conversion inside) of the UNMODIFIED reference
    engine with the CUDA plug-in selected, beside the same engine on its own CPU backend: median of >= 10 runs for config 1
    and for one config-2 encoder layer. The CPU backend takes about a minute per run on the full batch of 8 images, so
    its config-2 time is taken on one image (images are independent: the batch costs 8 times that)."""
    from oracle import vko
    from vknn_b200.synthetic import encoder_weights
    if not os.path.exists(vko.REF_DRIVER_CUDA):
        return {"unavailable": "the reference engine with the plug-in is not built here (oracle/_ref/vknn_ref_driver_cuda)"}
    out = {}
    try:
        rng = np.random.default_rng(1001)
        q, k, v = (rng.standard_normal((1, 12, 197, 64)).astype(np.float32) for _ in range(3))
        _, cuda = vko.attention_graph(q, k, v, 0.125).run(backend="cuda", precision="low", iters=20, warmup=3, timeout=300)
        _, cpu = vko.attention_graph(q, k, v, 0.125).run(backend="cpu", iters=10, warmup=1, timeout=300)
        out["config1_attention"] = {"cuda_session_run_ms": cuda["median_ms"], "cpu_session_run_ms": cpu["median_ms"], "runs": 20,
                                    "io": "host fp32 in / out, f16 storage on the device"}
        rng = np.random.default_rng(1002)
        w = encoder_weights(rng, 768, 3072)
        x = rng.standard_normal((8, 197, 768)).astype(np.float32)
        _, cuda = vko.encoder_layer_graph(x, w, 12).run(backend="cuda", precision="low", iters=20, warmup=3, tuning="fast", timeout=300)
        _, cpu = vko.encoder_layer_graph(x[:1], w, 12).run(backend="cpu", iters=1, warmup=0, timeout=300)
        out["config2_layer"] = {"cuda_session_run_ms": cuda["median_ms"], "tok_s": 8 * 197 / (cuda["median_ms"] * 1e-3), "runs": 20,
                                "cpu_session_run_ms_one_image": cpu["median_ms"], "cpu_tok_s": 197 / (cpu["median_ms"] * 1e-3),
                                "io": "host fp32 in / out (4.8 MB each way), fp16 weights and activations on the device"}
    except Exception as e:  # noqa: BLE001 - informational leg
        out["error"] = str(e)[:300]
    return out


# ---------------------------------------------------------------------------------------------------------------
def cpu_baseline_prefill(cfg, budget_rows=256):
    """Times the reference's own CPU backend (oracle/_ref, one core) on a bounded sample of the headline workload:
    `budget_rows` query rows of one (batch, head) unit against all S keys (rows are independent without a mask)."""
    from oracle import vko
    S, D = cfg["S"], cfg["D"]
    rng = np.random.default_rng(cfg["seed"])
    q = rng.standard_normal((1, 1, budget_rows, D)).astype(np.float32)
    k = rng.standard_normal((1, 1, S, D)).astype(np.float32)
    v = rng.standard_normal((1, 1, S, D)).astype(np.float32)
    flops = 4.0 * budget_rows * S * D
    sample = "%d query rows x %d keys of one (batch, head) unit, D=%d, fp32" % (budget_rows, S, D)
    if vko.have_ref():
        _, info = vko.attention_graph(q, k, v, 1.0 / np.sqrt(D)).run(iters=3, warmup=1)
        sec = info["median_ms"] * 1e-3
        kind = "reference"
    else:
        t0 = time.perf_counter()
        vko.attention(q, k, v, 1.0 / np.sqrt(D), threads=1)
        sec = time.perf_counter() - t0
        kind = "port"
    return {"value": flops / sec / 1e12, "unit": "TFLOP/s", "cores": 1, "kind": kind, "sample": sample, "seconds": sec}


def run_reference(args):
    """Reference arm: the reference's own CPU implementation of the path on the host cores (one process per core,
    each an unmodified single-threaded reference Session on its own slice of query rows)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    from concurrent.futures import ThreadPoolExecutor
    from oracle import vko
    cfg = PREFILL
    S, D = cfg["S"], cfg["D"]
    cores = max(1, min(os.cpu_count() or 1, 32))
    rows = 128
    flops_proc = 4.0 * rows * S * D
    kind = "reference" if vko.have_ref() else "port"

    def one(i):
        rng = np.random.default_rng(cfg["seed"] + i)
        q = rng.standard_normal((1, 1, rows, D)).astype(np.float32)
        k = rng.standard_normal((1, 1, S, D)).astype(np.float32)
        v = rng.standard_normal((1, 1, S, D)).astype(np.float32)
        if kind == "reference":
            _, info = vko.attention_graph(q, k, v, 1.0 / np.sqrt(D)).run(iters=args.steps, warmup=args.warmup)
            return info["median_ms"]
        for _ in range(args.warmup):
            vko.attention(q, k, v, 1.0 / np.sqrt(D), threads=1)
        ts = []
        for _ in range(args.steps):
            t0 = time.perf_counter()
            vko.attention(q, k, v, 1.0 / np.sqrt(D), threads=1)
            ts.append((time.perf_counter() - t0) * 1e3)
        return float(np.median(ts))

    with ThreadPoolExecutor(max_workers=cores) as ex:
        ms = list(ex.map(one, range(cores)))
    step_ms = max(ms)
    value = flops_proc * cores / (step_ms * 1e-3) / 1e12
    line = {
        "impl": "reference", "metric": "attention TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": headline_config(cfg, args.gpus),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": kind,
                         "sample": "per step: %d processes x %d query rows x %d keys of (batch, head) units, D=%d, fp32, reference CPU backend" %
                                   (cores, rows, S, D)},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))
    return 0


def headline_config(cfg, n, delivery=None):
    c = {"workload": "config 4: prefill attention, batch %d x %d heads, head_dim %d, seq %d, %s, %s" %
                     (cfg["B"], cfg["H"], cfg["D"], cfg["S"], cfg["dtype"], "causal" if cfg["causal"] else "no mask"),
         "parallelism": ("strong scaling: the one named configuration sharded by head over %d rank(s), %d heads per GPU" % (n, cfg["H"] // max(n, 1))) +
                        ("; the step ends when every rank holds the whole attention output [B, S, H*D] (all-gather at the "
                         "attention-output boundary inside the timed region)" if n > 1 else " (one GPU: nothing to deliver)"),
         "l2": "inputs cycle through sets larger than L2 (126 MB) between timed steps"}
    if delivery:
        c["delivery"] = delivery
    return c


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="prefill", choices=["prefill", "decode", "encoder", "layernorm"])
    ap.add_argument("--seq", type=int, default=None, help="prefill sequence length (default 8192)")
    ap.add_argument("--causal", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the decode / encoder / sweep extras")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline and plug-in legs")
    ap.add_argument("--no-tune", action="store_true", help="encoder workloads: keep the built-in GEMM configurations (no per-shape timing)")
    ap.add_argument("--cooldown", type=float, default=1.0, help="idle seconds before each leg of the prefill sweep and before the delivered step at N > 1")
    ap.add_argument("--sustained", type=float, default=2.2, help="seconds of the back-to-back run of the headline kernel (0: skip)")
    args = ap.parse_args()
    global NO_TUNE
    NO_TUNE = args.no_tune
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import vknn_b200
    rank, world, local = dist_setup(args.gpus)
    ctx = vknn_b200.Context(local)
    pk = peaks()
    cfg = dict(PREFILL)
    if args.seq:
        cfg["S"] = args.seq
    cfg["causal"] = bool(args.causal)
    if args.workload == "prefill" and cfg["H"] % world:
        raise SystemExit("the %d heads of the configuration do not divide over %d ranks" % (cfg["H"], world))

    sampler = None
    if rank == 0:
        try:
            uuid = "GPU-" + str(torch.cuda.get_device_properties(local).uuid)
        except Exception:  # noqa: BLE001
            uuid = None
        sampler = ClockSampler(local, uuid)
        sampler.start()
    strong = None
    if args.workload == "prefill":
        Hl = cfg["H"] // world
        r = bench_prefill(ctx, cfg, args.steps, args.warmup, rank, world, e2e_steps=args.steps, heads_per_rank=Hl,
                          sustained_s=args.sustained, sampler=sampler)
        if world > 1:
            # the delivered step is the headline at N > 1: like the one-GPU headline it starts from an idle GPU, not from the
            # power state the sustained leg above leaves behind
            import torch
            torch.cuda.synchronize()
            time.sleep(args.cooldown)
            barrier(world)
            strong = bench_prefill_delivered(ctx, cfg, args.steps, args.warmup, rank, world)
    elif args.workload == "decode":
        r = bench_decode(ctx, DECODE, args.steps, args.warmup, rank, world)
    elif args.workload == "layernorm":
        r = bench_layernorm(ctx, LAYERNORM, args.steps, args.warmup, rank, world)
    else:
        r = bench_encoder(ctx, ENCODER, args.steps, args.warmup, rank, world)
    if args.workload != "prefill":
        r["window"] = tuple(LAST_WINDOW)
    clocks = sampler.window(*r["window"]) if rank == 0 else None

    extra = {}
    if not args.no_extra:
        k = min(args.steps, 10)
        if args.workload != "decode":
            d = bench_decode(ctx, DECODE, k, 3, rank, world)
            extra["decode"] = {"workload": "config 5: GQA decode, batch 32, 32q/8kv heads, D=128, fp16 cache 8192, kv_len U[1024,8192], per rank (weak scaling, batch sharded)",
                               "GB/s": d["gbs"], "ms_per_step": d["total_ms"] / k,
                               "roofline": hbm_roofline(d["bytes_step_rank"], d["per_launch_ms"], pk, traffic=NCU_DECODE_DRAM_OVER_ALGORITHMIC * d["bytes_step_rank"],
                                                        kernel="attn_decode_tc_kernel (+ attn_decode_combine_kernel)")}
            extra["decode"]["frac_hbm_per_gpu"] = extra["decode"]["roofline"]["frac"]
            if world > 1 and DECODE["B"] % world == 0:
                ds = bench_decode(ctx, DECODE, k, 3, rank, world, strong=True)
                extra["decode_strong"] = {"workload": "config 5, the one batch of 32 sequences sharded by batch, %d per rank, no collective" % (DECODE["B"] // world),
                                          "GB/s": ds["gbs"], "ms_per_step": ds["total_ms"] / k,
                                          "roofline": hbm_roofline(ds["bytes_step_rank"], ds["per_launch_ms"], pk, kernel="attn_decode_tc_kernel (+ combine)",
                                                                   note="rank 0's shard; the launch is short enough that launch latency shows")}
        if args.workload != "encoder":
            e = bench_encoder(ctx, ENCODER, k, 3, rank, world)
            extra["encoder"] = {"workload": "config 2: ViT-B/16 layer, batch 8 x 197 tokens per rank, fp16 (weak scaling, batch sharded)", "tok/s": e["tok_s"],
                                "TFLOP/s": e["tflops"], "ms_per_step": e["total_ms"] / k,
                                "roofline": tensor_roofline(e["flops_step_rank"], e["per_launch_ms"], pk, kernel="7 launches: layernorm, gemm_tcgen05 x4, attn_prefill, layernorm")}
        if args.workload == "prefill" and not args.seq:
            st = bench_stack(ctx, STACK, max(3, k // 3), 3, rank, world)
            st["roofline"] = tensor_roofline(st.pop("flops_step_rank"), st.pop("per_launch_ms"), pk, kernel="192 launches per forward (24 layers)")
            extra["encoder_stack"] = dict(st, workload="config 3: 24 layers, d=1024, 16 heads, MLP 4096, 2738 tokens, batch 1 per rank, fp16")
        if args.workload != "layernorm":
            ln = bench_layernorm(ctx, LAYERNORM, k, 3, rank, world)
            extra["layernorm"] = {"workload": "LayerNorm over 131072 rows x 1024 (config 3 width), fp16, replicated per rank",
                                  "roofline": hbm_roofline(ln["bytes_step_rank"], ln["per_launch_ms"], pk, traffic=float(ln["bytes_step_rank"]), kernel="layernorm_kernel")}
            extra["layernorm"]["GB/s_per_gpu"] = extra["layernorm"]["roofline"]["achieved"]
            extra["layernorm"]["frac_hbm_per_gpu"] = extra["layernorm"]["roofline"]["frac"]
        if args.workload == "prefill" and not args.seq:
            rs = bench_raster(ctx, max(3, k // 2), 3, rank, world)
            rs["roofline"] = hbm_roofline(rs["algorithmic_bytes"], rs["ms_per_view_f64"], pk, kernel="raster_* (5 kernels)",
                                          note="a few MB per view: the pass is bound by sort and compositing latency, not by HBM")
            extra["raster"] = rs
        if args.workload == "prefill" and not args.seq:
            sweep, weak = {}, {}
            n = max(5, k)
            for S, causal in ((4096, False), (16384, False), (8192, True), (16384, True)):
                c2 = dict(cfg, S=S, causal=causal)
                # Like the headline, each leg is a burst from an idle GPU: after tens of milliseconds of back-to-back attention
                # launches the power management already holds the kernel back (seq 8192 causal: 0.90 ms per launch from idle,
                # 1.05 ms right after forty launches of the unmasked shape, the sampled clock still at its maximum).
                import torch
                torch.cuda.synchronize()
                time.sleep(args.cooldown)
                barrier(world)
                s = bench_prefill(ctx, c2, n, 3, rank, world)
                name = "S%d%s" % (S, "_causal" if causal else "")
                tf = s["flops_step_rank"] * world * n / (s["total_ms"] * 1e-3) / 1e12
                sweep[name] = {"TFLOP/s": tf, "roofline": tensor_roofline(s["flops_step_rank"], s["per_launch_ms"], pk, kernel="attn_prefill_kernel",
                                                                         traffic=NCU_PREFILL_DRAM_BYTES_PER_ROW_UNIT * c2["B"] * c2["H"] * S)}
                if rank == 0:  # these legs run late in a long job: say at which clock and under which cap they were taken
                    w = sampler.window(*s["window"])
                    sweep[name]["clocks"] = {"sm_mhz": w["sm_mhz"], "reasons": w["reasons"], "power_w_max": w.get("power_w_max"), "samples": w["samples"]}
                    sweep[name]["roofline"]["frac_of_sustained"] = sweep[name]["roofline"]["achieved"] / pk["bf16_tflops_sustained"]
            extra["prefill_sweep"] = dict(sweep, cooldown_s=args.cooldown,
                                          note="every rank runs the whole named configuration (weak scaling); aggregate TFLOP/s, per-launch roofline of rank 0; "
                                               "the GPU idles cooldown_s before each leg, so each is a burst like the headline")
            if world > 1:
                s = bench_prefill(ctx, cfg, n, 3, rank, world)
                weak["prefill_TFLOP/s"] = s["flops_step_rank"] * world * n / (s["total_ms"] * 1e-3) / 1e12
                weak["note"] = "every rank runs the whole named configuration, outputs left sharded, no collective: N independent GPUs"
                weak["decode_GB/s"] = extra["decode"]["GB/s"]
                weak["encoder_tok/s"] = extra["encoder"]["tok/s"]
                weak["encoder_stack_tok/s"] = extra["encoder_stack"]["tok_s"]
                extra["weak"] = weak
    if sampler:
        sampler.stop()
    if rank != 0:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()
        return 0
    line = {"n_gpus": world, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "vs_baseline": None, "data": "synthetic",
            "clocks": clocks, "extra": extra}
    if args.workload == "prefill":
        flops_cfg = prefill_flops(cfg, cfg["H"])
        attn_ms = r["total_ms"] / args.steps  # attention alone on this rank's heads, max over ranks
        step_ms, delivery, launches = attn_ms, None, int(r["launches"])
        if strong:
            best = None
            for name in ("nccl_allgather", "fused_fanout"):
                s = strong.get(name, {})
                if "ms_per_step" in s:
                    s["TFLOP/s"] = flops_cfg / (s["ms_per_step"] * 1e-3) / 1e12
                    s["delivery_share_of_step"] = max(0.0, 1.0 - attn_ms / s["ms_per_step"])
                    if best is None or s["ms_per_step"] < strong[best]["ms_per_step"]:
                        best = name
            step_ms, delivery = strong[best]["ms_per_step"], best
            gather_bytes = cfg["B"] * cfg["S"] * cfg["H"] * cfg["D"] * 2 * (world - 1) // world  # received per rank
            strong["attention_only_ms"] = attn_ms
            strong["attention_only_TFLOP/s"] = flops_cfg / (attn_ms * 1e-3) / 1e12
            strong["gather_bytes_received_per_rank"] = gather_bytes
            strong["gather_GB/s_per_rank_if_serial"] = gather_bytes / max((step_ms - attn_ms) * 1e-3, 1e-9) / 1e9
            units = cfg["B"] * r["heads_per_rank"] * ((cfg["S"] + 255) // 256)
            strong["limits"] = "per rank %d two-tile CTAs on 148 SMs (%.2f waves); every rank receives %.0f MB per step over NVLink (%.3f ms at the measured " \
                               "725 GB/s all-gather bus bandwidth) against %.3f ms of attention" % (units, units / 148.0, gather_bytes / 1e6, gather_bytes / 725e9 * 1e3, attn_ms)
            extra["strong"] = strong
            launches = args.steps * (2 if delivery == "fused_fanout" else 1)
        value = flops_cfg / (step_ms * 1e-3) / 1e12
        roof = tensor_roofline(r["flops_step_rank"], r["per_launch_ms"], pk, kernel="attn_prefill_kernel",
                               traffic=NCU_PREFILL_DRAM_BYTES_PER_ROW_UNIT * cfg["B"] * r["heads_per_rank"] * cfg["S"],
                               traffic_note="ncu capture at seq 2048 scaled by (batch, head, query row) units; algorithmic bytes %d" % r["bytes_step_rank"],
                               frac_of_sustained=r["flops_step_rank"] / (r["per_launch_ms"] * 1e-3) / 1e12 / pk["bf16_tflops_sustained"],
                               flops_per_launch=r["flops_step_rank"])
        if "sustained" in r:
            s = r["sustained"]
            s["frac_of_sustained_peak"] = s["tflops"] / pk["bf16_tflops_sustained"]
            s["tflops_x_mhz"] = s["tflops"] / s["sm_mhz_median"] * (clocks["sm_max_mhz"] or 1965.0) if s.get("sm_mhz_median") else None
            s["note"] = "the same launch back to back between two events; frac against the sustained cuBLAS figure; tflops_x_mhz = the rate rescaled to the maximum SM clock"
            roof["sustained"] = s
        line.update({"metric": "attention TFLOP/s", "value": value, "unit": "TFLOP/s", "ms_per_step": step_ms, "scaling": "strong", "dtype": "bf16",
                     "config": headline_config(cfg, world, delivery), "gpu_launches": launches, "roofline": roof})
        if "e2e_ms_per_step" in r:
            line["e2e"] = {"value": flops_cfg / (r["e2e_ms_per_step"] * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": int(r["h2d"]),
                           "d2h_bytes_per_step": int(r["d2h"]), "ms_per_step": r["e2e_ms_per_step"], "steps": r["e2e_steps"],
                           "note": "every rank uploads the Q/K/V of its heads from pinned host memory and downloads its heads of O; bytes are whole-job totals"}
    elif args.workload == "decode":
        line.update({"metric": "decode GB/s", "value": r["gbs"], "unit": "GB/s", "ms_per_step": r["total_ms"] / args.steps, "scaling": "weak",
                     "dtype": "f16", "config": {"workload": "config 5: GQA decode batch 32, 32q/8kv heads, D=128, cache 8192", "parallelism": "weak scaling: the named configuration per rank, sharded by batch, no collective"},
                     "gpu_launches": 2 * args.steps,
                     "roofline": hbm_roofline(r["bytes_step_rank"], r["per_launch_ms"], pk, traffic=NCU_DECODE_DRAM_OVER_ALGORITHMIC * r["bytes_step_rank"],
                                              kernel="attn_decode_tc_kernel (+ attn_decode_combine_kernel)")})
    elif args.workload == "layernorm":
        line.update({"metric": "layernorm GB/s", "value": r["gbs"], "unit": "GB/s", "ms_per_step": r["total_ms"] / args.steps, "scaling": "weak",
                     "dtype": "f16", "config": {"workload": "LayerNorm 131072 rows x 1024, fp16", "parallelism": "replicated"},
                     "gpu_launches": args.steps,
                     "roofline": hbm_roofline(r["bytes_step_rank"], r["per_launch_ms"], pk, traffic=float(r["bytes_step_rank"]), kernel="layernorm_kernel")})
    else:
        line.update({"metric": "encoder tok/s", "value": r["tok_s"], "unit": "tok/s", "ms_per_step": r["total_ms"] / args.steps, "scaling": "weak",
                     "dtype": "f16", "config": {"workload": "config 2: ViT-B/16 encoder layer batch 8 x 197", "parallelism": "weak scaling: the named configuration per rank, sharded by batch, no collective"},
                     "gpu_launches": 7 * args.steps,
                     "roofline": tensor_roofline(r["flops_step_rank"], r["per_launch_ms"], pk)})
    if world == 1 and not args.no_cpu and args.workload == "prefill":
        try:
            line["cpu_baseline"] = cpu_baseline_prefill(cfg)
        except Exception as e:  # the baseline is informational; its failure must not hide the GPU numbers
            line["cpu_baseline"] = {"value": None, "unit": "TFLOP/s", "cores": 1, "kind": "unavailable", "sample": str(e)[:200]}
        if not args.no_extra and not args.seq:
            ctx.sync()
            extra["plugin_e2e"] = plugin_e2e()
    print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
