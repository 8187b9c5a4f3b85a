#!/usr/bin/env python
"""LayerAdam throughput benchmark.

    python bench.py [--gpus N] [--steps K] [--warmup W]            # the CUDA path
    python bench.py --impl reference [--gpus N] [--steps K] [--warmup W]   # the reference's CPU kernel

A step is one LayerAdam update of one Llama-3.1-8B decoder layer flattened to 218,112,000
fp32 parameters (bf16 gradient in, fp32 p / m / v updated in place, bf16 copy out): 28
algorithmic bytes per parameter.  Synthetic data with the layer's value distributions.

N = 1   state resident in HBM, one launch per step.
N > 1   launched by torchrun, one rank per GPU: each rank brings its own full-layer bf16
        gradient, owns 1/N of p / m / v, the gradients are averaged in fp32 in rank order
        (fused peer reads, or NCCL reduce-scatter with --dp-mode nccl), the shard is updated
        and the bf16 shards are all-gathered.  The layer size is fixed, so scaling is strong.

Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

N_LAYER = 218_112_000  # q/o 4096x4096, k/v 4096x1024, gate/up/down 4096x14336, two 4096 norms
BYTES_PER_PARAM = 28   # read p4 + g2 + m4 + v4, write p4 + m4 + v4 + bf16 2
HP = dict(lr=1e-5, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
WORKLOAD = "llama3.1-8b decoder layer, flat n=218112000, fp32 p/m/v + bf16 grad -> bf16 copy"
METRIC = "LayerAdam Gparams/s"
FALLBACK_HBM_GBS = 6650.0
L2_BYTES = 126e6
SWEEP_SIZES = (1_000_448, 16_000_000, N_LAYER, 1_000_000_512)   # "1M, 16M, 218M, 1B", multiples of 128 * 8


# dram__bytes_read.sum + dram__bytes_write.sum per launch of adam_vec4_kernel as ncu captured them
# (a profiler cannot run inside a timed benchmark, so this is carried over, not re-measured): at
# n = 218,112,000 reads are 3,053.7 MB (14.00 B/param) and writes 2,993.5 MB, i.e. 14 B/param
# minus about 60 MB that is still dirty in L2 when the kernel ends (the same shortfall, 53-57 MB,
# shows at n = 16,777,216: it does not grow with n).  Scaled to a launch over `units` parameters.
def ncu_traffic_bytes(units: int) -> float:
    return 14.0 * units + max(14.0 * units - 60e6, 0.0)


_RESULT_FD = None
T_START = time.perf_counter()


def emit(line: str) -> None:
    """Write the result line to the real stdout (see main)."""
    data = (line + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(line + "\n")
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def measured_peak():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            return float(json.loads(f.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


# ---------------------------------------------------------------------------------------------
# clocks: read-only NVML sampling in a thread while the GPU is under load
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
               0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}

    def __init__(self, torch_index: int, period_s: float = 0.004):
        self.samples = []  # (t, sm_mhz, reasons_mask, in_timed_region)
        self.period = period_s
        self.in_region = False
        self._stop = threading.Event()
        self.ok = False
        self.sm_max = None
        try:
            import pynvml
            import torch
            self.nv = pynvml
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(torch_index).uuid)
            h = None
            for i in range(pynvml.nvmlDeviceGetCount()):
                hi = pynvml.nvmlDeviceGetHandleByIndex(i)
                u = pynvml.nvmlDeviceGetUUID(hi)
                u = u.decode() if isinstance(u, bytes) else u
                if uuid in u:
                    h = hi
                    break
            self.h = h if h is not None else pynvml.nvmlDeviceGetHandleByIndex(torch_index)
            self.sm_max = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception as exc:  # NVML not reachable: report that instead of clocks
            self.err = repr(exc)
        self.thread = threading.Thread(target=self._run, daemon=True)

    def _read(self):
        nv = self.nv
        sm = int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
        try:
            mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
        except Exception:
            mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
        return sm, mask

    def _run(self):
        while not self._stop.is_set():
            try:
                sm, mask = self._read()
                self.samples.append((time.perf_counter(), sm, mask, self.in_region))
            except Exception:
                pass
            time.sleep(self.period)

    def start(self):
        if self.ok:
            self.thread.start()

    def stop(self):
        self._stop.set()
        if self.ok and self.thread.is_alive():
            self.thread.join(timeout=2)

    def summary(self):
        if not self.ok:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "note": "NVML unavailable: " + getattr(self, "err", "")}
        timed = [s for s in self.samples if s[3]]
        used, scope = (timed, "timed region") if len(timed) >= 3 else ([s for s in self.samples], "whole loaded run (timed region too short to sample)")
        if not used:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": [], "note": "no samples"}
        mask = 0
        for s in used:
            mask |= s[2]
        reasons = [name for bit, name in self.REASONS.items() if mask & bit and name != "gpu_idle"]
        return {"sm_mhz": statistics.median(s[1] for s in used), "sm_max_mhz": self.sm_max, "reasons": reasons,
                "samples": len(used), "scope": scope}


# ---------------------------------------------------------------------------------------------
# CPU arms (the reference's kernel when its prebuilt module is present, else the C port)
# ---------------------------------------------------------------------------------------------
def cpu_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def run_cpu_arm(n: int, steps: int, warmup: int, budget_s: float):
    """Time the CPU LayerAdam step on this host with all usable threads.
    Returns dict(value=Gparams/s, kind, cores, sample, ms_per_step, steps)."""
    import numpy as np
    import torch
    threads = cpu_threads()
    os.environ.setdefault("OMP_NUM_THREADS", str(threads))
    torch.set_num_threads(threads)
    from oracle import build_ref
    ref = build_ref.load()
    gen = torch.Generator().manual_seed(0)
    p = torch.empty(n).normal_(0, 0.02, generator=gen)
    p[-8192:] = 1.0
    m, v = torch.zeros(n), torch.zeros(n)
    grads = [torch.empty(n).normal_(0, 1e-3, generator=gen).to(torch.bfloat16) for _ in range(2)]
    lr, (b1, b2), eps, wd = HP["lr"], HP["betas"], HP["eps"], HP["weight_decay"]
    if ref is not None:
        kind = "reference"
        ref.create_adam(0, lr, b1, b2, eps, wd, True, False)

        def one(step):
            ref.adam_update(0, step, lr, b1, b2, eps, wd, True, p, grads[step & 1], m, v)
    else:
        kind = "port"
        from oracle import oracle as O
        opt = O.OracleAdam(lr, b1, b2, eps, wd, True)
        pn, mn, vn = p.numpy(), m.numpy(), v.numpy()
        gn = [g.view(torch.int16).numpy().view(np.uint16) for g in grads]

        def one(step):
            opt.adam_update(step, lr, b1, b2, eps, wd, True, pn, gn[step & 1], mn, vn)
    step = 0
    t_w0 = time.perf_counter()
    for _ in range(max(1, warmup)):
        step += 1
        one(step)
    per = (time.perf_counter() - t_w0) / max(1, warmup)
    steps = max(1, min(steps, int(budget_s / max(per, 1e-6))))
    t0 = time.perf_counter()
    for _ in range(steps):
        step += 1
        one(step)
    dt = time.perf_counter() - t0
    # the reference converts fp32 -> bf16 in a separate CPU pass before the upload
    # (transformer_layer.py:296-305); time it too, it is part of what the fused kernel replaces
    stage = torch.empty(n, dtype=torch.bfloat16)
    t1 = time.perf_counter()
    for _ in range(2):
        stage.copy_(p)
    cast_ms = (time.perf_counter() - t1) / 2 * 1e3
    return dict(value=n * steps / dt / 1e9, unit="Gparams/s", cores=threads, kind=kind,
                sample=f"{steps} full-layer steps (n={n}) after {max(1, warmup)} warm-up, bf16 grad, all host threads; "
                       f"separate fp32->bf16 cast pass {cast_ms:.1f} ms not included",
                ms_per_step=dt / steps * 1e3, steps=steps, bf16_cast_ms=cast_ms)


def main_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    r = run_cpu_arm(args.n, args.steps, args.warmup, budget_s=90.0)
    line = {"impl": "reference", "metric": METRIC, "value": r["value"], "unit": "Gparams/s", "n_gpus": args.gpus,
            "steps": r["steps"], "warmup": max(1, args.warmup), "ms_per_step": r["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": {"workload": WORKLOAD, "where": "host CPU"},
            "cpu_baseline": {"value": r["value"], "unit": "Gparams/s", "cores": r["cores"], "kind": r["kind"],
                             "sample": r["sample"]},
            "e2e": {"value": r["value"], "unit": "Gparams/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    emit(json.dumps(line))
    return 0


# ---------------------------------------------------------------------------------------------
# parity inside the benchmark: a few more steps, checked against the CPU oracle
# ---------------------------------------------------------------------------------------------
def _window_starts(a: int, b: int, width: int):
    """Up to three [lo, hi) windows of [a, b): at the start, around the middle, at the end;
    starts on multiples of 16 elements relative to the layer."""
    k = b - a
    if k <= 0:
        return []
    w = min(width, k)
    lows = {a, a + ((k - w) // 2) // 16 * 16, max(a, (b - w) // 16 * 16)}
    return sorted((lo, min(lo + w, b)) for lo in lows)


def _rel_vec_n(n: int, lo: int, hi: int) -> int:
    return min(max((n & ~15) - lo, 0), hi - lo)


def parity_single(dev, p, m, v, out, grads, n, steps=3, width=1 << 16):
    """N = 1: `steps` more updates with a fresh optimizer object (so the scalar call history is
    known), three windows of p / m / v / bf16 compared with the oracle bit for bit."""
    import numpy as np
    import torch
    from oracle import oracle as O
    from slideformer_b200 import LayerAdam
    hp = (HP["lr"], HP["betas"][0], HP["betas"][1], HP["eps"], HP["weight_decay"])
    opt = LayerAdam(**HP)
    orc = O.OracleAdam(*hp, True)
    group = dict(opt.defaults, step=0)
    wins = _window_starts(0, n, width)
    cpu = [[t[lo:hi].cpu().numpy().copy() for t in (p, m, v)] + [np.zeros(hi - lo, np.uint16)] for lo, hi in wins]
    for j in range(steps):
        group["step"] += 1
        g = grads[j % len(grads)]
        opt.step_chunk(p, g, m, v, group, out)
        c = orc.scalars(group["step"], *hp, True)
        for (lo, hi), (pw, mw, vw, ow) in zip(wins, cpu):
            gw = g[lo:hi].view(torch.int16).cpu().numpy().view(np.uint16)
            O.apply_step(c, pw, gw, mw, vw, ow, vec_n=_rel_vec_n(n, lo, hi))
    torch.cuda.synchronize()
    elems = mism = 0
    for (lo, hi), (pw, mw, vw, ow) in zip(wins, cpu):
        for want, got in ((pw, p), (mw, m), (vw, v)):
            mism += int((got[lo:hi].cpu().numpy().view(np.uint32) != want.view(np.uint32)).sum())
            elems += hi - lo
        mism += int((out[lo:hi].view(torch.int16).cpu().numpy().view(np.uint16) != ow).sum())
        elems += hi - lo
    return {"elements": elems, "mismatches": mism, "steps": steps, "windows": [list(w) for w in wins],
            "what": "p, m, v and the bf16 copy after extra steps vs the CPU oracle, bit for bit"}


def parity_sharded(sh, world, rank, dev, steps=3, width=1 << 16):
    """N > 1: `steps` more sharded steps with a fresh optimizer object; for three windows of every
    rank's owned slice the ranks' gradients are all-gathered, the oracle computes the fp32
    rank-order mean and the reference update, and (a) the owner's p / m / v and (b) EVERY rank's
    pushed bf16 copy of that window are compared bit for bit.  Totals are summed over ranks."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from oracle import oracle as O
    from slideformer_b200 import LayerAdam
    from slideformer_b200.shared_data_parallel import shard_range
    hp = (HP["lr"], HP["betas"][0], HP["betas"][1], HP["eps"], HP["weight_decay"])
    sh.adam = LayerAdam(**HP)
    sh.group = dict(sh.adam.defaults, step=0)
    orc = O.OracleAdam(*hp, True)
    st, dp, n = sh.state, sh.dp, sh.numel
    wins = {r: _window_starts(*shard_range(n, world, r), width) for r in range(world)}
    a0 = st.start
    cpu = [[t[lo - a0:hi - a0].cpu().numpy().copy() for t in (st.params, st.exp_avg, st.exp_avg_sq)]
           + [np.zeros(hi - lo, np.uint16)] for lo, hi in wins[rank]]
    for j in range(steps):
        slot = j % dp.exchange_slots
        sh.step(slot)
        mine_rows = []
        for r in range(world):
            for lo, hi in wins[r]:
                local = dp.grad_buffer(slot)[lo:hi].contiguous()
                rows = [torch.empty_like(local) for _ in range(world)]
                dist.all_gather(rows, local)
                if r == rank:
                    mine_rows.append(np.stack([x.view(torch.int16).cpu().numpy().view(np.uint16) for x in rows]))
        c = orc.scalars(sh.group["step"], *hp, True)
        for (lo, hi), rows, (pw, mw, vw, ow) in zip(wins[rank], mine_rows, cpu):
            O.apply_step(c, pw, O.rank_mean(rows), mw, vw, ow, vec_n=_rel_vec_n(n, lo, hi))
    torch.cuda.synchronize()
    elems = mism = 0
    for (lo, hi), (pw, mw, vw, ow) in zip(wins[rank], cpu):
        for want, got in ((pw, st.params), (mw, st.exp_avg), (vw, st.exp_avg_sq)):
            mism += int((got[lo - a0:hi - a0].cpu().numpy().view(np.uint32) != want.view(np.uint32)).sum())
            elems += hi - lo
    for r in range(world):                      # the pushed bf16 layer, on every rank
        for wi, (lo, hi) in enumerate(wins[r]):
            exp = (torch.from_numpy(cpu[wi][3].astype(np.int32)).to(dev) if r == rank
                   else torch.empty(hi - lo, dtype=torch.int32, device=dev))
            dist.broadcast(exp, src=r)
            if st.bf16 is not None:
                got = st.bf16[lo:hi].view(torch.int16).to(torch.int32) & 0xFFFF
                mism += int((got != exp).sum().item())
                elems += hi - lo
    t = torch.tensor([elems, mism], dtype=torch.int64, device=dev)
    dist.all_reduce(t)
    return {"elements": int(t[0]), "mismatches": int(t[1]), "steps": steps, "windows_per_rank": len(wins[rank]),
            "what": "owned p, m, v slices and every rank's pushed bf16 layer after extra sharded steps vs the CPU "
                    "oracle fed with the all-gathered gradients (fp32 rank-order mean), bit for bit"}


# ---------------------------------------------------------------------------------------------
# the standalone Adam-step sweep (1M / 16M / 218M / 1B flat vectors)
# ---------------------------------------------------------------------------------------------
def sweep_single(dev, peak, main_entry):
    """HBM-resident single-GPU step at each size.  Sizes whose working set fits in the L2 rotate
    through enough independent (p, g, m, v, out) sets that every launch finds its data in HBM."""
    import math
    import torch
    from slideformer_b200 import LayerAdam
    rows = []
    for ns in SWEEP_SIZES:
        if ns == main_entry["n"]:
            rows.append(main_entry)
            continue
        sets = max(1, min(64, math.ceil(4 * L2_BYTES / (BYTES_PER_PARAM * ns))))
        gen = torch.Generator(device=dev).manual_seed(ns % 9973)
        state = []
        for _ in range(sets):
            p = torch.empty(ns, device=dev).normal_(0, 0.02, generator=gen)
            g = torch.empty(ns, device=dev).normal_(0, 1e-3, generator=gen).to(torch.bfloat16)
            state.append((p, g, torch.zeros(ns, device=dev), torch.zeros(ns, device=dev),
                          torch.empty(ns, device=dev, dtype=torch.bfloat16)))
        opt = LayerAdam(**HP)
        group = dict(opt.defaults, step=0)

        def one(i):
            p, g, m, v, o = state[i % sets]
            group["step"] += 1
            opt.step_chunk(p, g, m, v, group, o)
        for i in range(max(3, sets)):
            one(i)
        torch.cuda.synchronize()
        est_ms = max(BYTES_PER_PARAM * ns / (peak * 1e9) * 1e3, 0.004)
        reps = int(min(max(100.0 / est_ms, 20), 2000))       # about 0.1 s of launches
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(reps):
            one(i)
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / reps
        gbs = BYTES_PER_PARAM * ns / (ms * 1e-3) / 1e9
        row = {"n": ns, "ms": ms, "gparams_per_s": ns / (ms * 1e-3) / 1e9, "hbm_gbs": gbs, "frac": gbs / peak,
               "launches": reps, "state_sets": sets,
               "l2": "rotating sets exceed L2" if sets > 1 else "inputs exceed L2"}
        if est_ms < 0.1:
            # a launch this short is bound by the host's launch rate; the same launches replayed from
            # a CUDA graph show what the GPU itself needs per launch
            try:
                graph = torch.cuda.CUDAGraph()
                per_graph = max(sets, 16)
                with torch.cuda.graph(graph):
                    for i in range(per_graph):
                        one(i)
                graph.replay()
                torch.cuda.synchronize()
                greps = max(3, reps // per_graph)
                a.record()
                for _ in range(greps):
                    graph.replay()
                b.record()
                torch.cuda.synchronize()
                gms = a.elapsed_time(b) / (greps * per_graph)
                row.update({"graph_ms": gms, "graph_hbm_gbs": BYTES_PER_PARAM * ns / (gms * 1e-3) / 1e9,
                            "graph_frac": BYTES_PER_PARAM * ns / (gms * 1e-3) / 1e9 / peak})
                del graph
            except Exception as exc:   # report, do not fail the benchmark over an optional figure
                row["graph_ms"] = None
                row["graph_note"] = repr(exc)[:200]
        rows.append(row)
        del state
        torch.cuda.empty_cache()
    return rows


def sweep_sharded(dev, world, mode, main_entry):
    """The sharded step at each size: kernel alone (with its NVLink traffic) and the whole step
    with its two cross-rank stream barriers.  Below a few million elements the step is bound by
    the barriers' latency, not by bytes, and nothing is flushed between launches."""
    import torch
    from slideformer_b200.shared_data_parallel import ShardedLayerAdam
    rows = []
    for ns in SWEEP_SIZES:
        if ns == main_entry["n"]:
            rows.append(main_entry)
            continue
        sh = ShardedLayerAdam(numel=ns, device=dev, mode=mode, **HP)
        gen = torch.Generator(device=dev).manual_seed(ns % 9973 + sh.dp.rank)
        sh.params_shard.normal_(0, 0.02, generator=gen)
        for k in range(3):
            sh.grad_buffer(k).normal_(0, 1e-3, generator=gen)
        for k in range(3):
            sh.step(k)
        kern_ms = sh.time_kernel_only(50)
        cnt = [0]

        def step():
            cnt[0] += 1
            sh.step(cnt[0] % 3)
        step_ms = sh._timed(step, 50)
        link = 2 * (world - 1) * sh.shard_numel * 2
        rows.append({"n": ns, "ms": step_ms, "kernel_ms": kern_ms, "gparams_per_s": ns / (step_ms * 1e-3) / 1e9,
                     "nvlink_gbs_per_direction": link / (kern_ms * 1e-3) / 1e9,
                     "frac": link / (kern_ms * 1e-3) / 1e9 / 770.0, "launches": 50,
                     "l2": "not flushed" if BYTES_PER_PARAM * ns / world < 4 * L2_BYTES else "inputs exceed L2"})
        sh.close()
        del sh
        torch.cuda.empty_cache()
    return rows


def fast_mode_nvls(sh, dev, world, n, reps=50):
    """The NVLS variant beside the exact one: same layer, gradients reduced and weights
    replicated inside the NVSwitch.  Reports its step time and how far three steps drift from
    the exact kernel started from the same state and gradients."""
    import torch
    import torch.distributed as dist
    from slideformer_b200 import LayerAdam
    from slideformer_b200.shared_data_parallel import ShardedLayerAdam
    try:
        from torch._C._distributed_c10d import _SymmetricMemory
        ok = bool(_SymmetricMemory.has_multicast_support(torch._C._autograd.DeviceType.CUDA, dev.index))
    except Exception:
        ok = False
    flags = [None] * world
    dist.all_gather_object(flags, ok)
    if not all(flags):
        return {"mode": "nvls", "unavailable": "the driver reports no NVLink multicast support on at least one GPU"}
    try:
        fast = ShardedLayerAdam(numel=n, device=dev, mode="nvls", **HP)
    except Exception as exc:
        return {"mode": "nvls", "unavailable": repr(exc)[:300]}
    ex_st, fa_st = sh.state, fast.state
    k = ex_st.end - ex_st.start
    for slot in range(3):
        fast.grad_buffer(slot).copy_(sh.grad_buffer(slot))
    # timing first (state drifts, which does not matter for time)
    fa_st.params.copy_(ex_st.params)
    for slot in range(3):
        fast.step(slot)
    kern_ms = fast.time_kernel_only(reps)
    cnt = [0]

    def step():
        cnt[0] += 1
        fast.step(cnt[0] % 3)
    step_ms = fast._timed(step, reps)
    # accuracy: both modes from one state, three steps, fresh optimizer objects
    start = ex_st.params.clone()
    for obj, st in ((sh, ex_st), (fast, fa_st)):
        st.params.copy_(start)
        st.exp_avg.zero_()
        st.exp_avg_sq.zero_()
        obj.adam = LayerAdam(**HP)
        obj.group = dict(obj.adam.defaults, step=0)
        for slot in range(3):
            obj.step(slot)
    torch.cuda.synchronize(dev)
    dp_abs = (fa_st.params[:k] - ex_st.params[:k]).abs().max() if k else torch.zeros((), device=dev)
    m_ref = ex_st.exp_avg[:k].abs().max().clamp(min=1e-30) if k else torch.ones((), device=dev)
    m_err = (fa_st.exp_avg[:k] - ex_st.exp_avg[:k]).abs().max() / m_ref if k else torch.zeros((), device=dev)
    same = (fa_st.params[:k].view(torch.int32) == ex_st.params[:k].view(torch.int32)).float().mean() if k else torch.ones((), device=dev)
    bf_same = (fast.state.bf16[:n].view(torch.int16) == sh.state.bf16[:n].view(torch.int16)).float().mean()
    t = torch.stack([dp_abs.float(), m_err.float()])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    u = torch.stack([same.float(), bf_same.float()])
    dist.all_reduce(u, op=dist.ReduceOp.MIN)
    received = 2 * fast.shard_numel * (world - 1) + 2 * fast.shard_numel   # pushed weights + reduced gradients
    out = {"mode": "nvls", "exact": False, "parallelism": fast.describe(), "ms_per_step": step_ms, "kernel_ms": kern_ms,
           "value": n / (step_ms * 1e-3) / 1e9, "unit": "Gparams/s",
           "dp_gradient_gparams_per_s": world * n / (step_ms * 1e-3) / 1e9,
           "nvlink_bytes_received_per_launch": received,
           "nvlink_gbs_received": received / (kern_ms * 1e-3) / 1e9,
           "accuracy_vs_exact": {"steps": 3, "max_abs_param_difference": float(t[0]),
                                 "max_abs_param_difference_over_lr": float(t[0]) / HP["lr"],
                                 "max_exp_avg_difference_over_max_exp_avg": float(t[1]),
                                 "min_fraction_of_fp32_params_bit_identical": float(u[0]),
                                 "min_fraction_of_bf16_weights_bit_identical": float(u[1])}}
    fast.close()
    return out


def measure_nvlink(dp, dev, nbytes: int = 1 << 29, reps: int = 10) -> dict:
    """What a bare copy kernel reaches between these GPUs (GB/s per direction per GPU): one GPU
    storing to its neighbour with the rest idle, every GPU storing to its neighbour at once,
    every GPU loading from its neighbour at once, and both at once (the traffic mix of the fused
    pull + push kernel: reads and writes in both directions of every link)."""
    import ctypes as C
    import torch
    import torch.distributed as dist
    from slideformer_b200 import _lib
    lib = _lib.load()
    base, peers = dp._shared_alloc(2 * nbytes)
    nxt = peers[(dp.rank + 1) % dp.world_size]
    src = torch.empty(nbytes, dtype=torch.uint8, device=dev).zero_()
    dst = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    s2 = torch.cuda.Stream(dev)

    def timed(push: bool, pull: bool, only_rank0: bool = False) -> float:
        active = (dp.rank == 0) or not only_rank0
        def once():
            if not active:
                return
            cur = torch.cuda.current_stream(dev)
            if push:
                _lib.check(lib.sf_copy_bytes(nxt, src.data_ptr(), nbytes, cur.cuda_stream))
            if pull:
                st = s2 if push else cur
                if push:
                    s2.wait_stream(cur)
                _lib.check(lib.sf_copy_bytes(dst.data_ptr(), nxt + nbytes, nbytes, st.cuda_stream))
        once()
        torch.cuda.synchronize(dev)
        dist.barrier()
        torch.cuda.synchronize(dev)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            once()
        torch.cuda.current_stream(dev).wait_stream(s2)
        b.record()
        torch.cuda.synchronize(dev)
        t = torch.tensor([a.elapsed_time(b) / reps if active else 0.0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        # bytes that crossed each direction of a GPU's links: its stores leave it, its loads enter
        # it, and with every GPU doing both each direction carries one copy of each kind
        per_direction = nbytes * (2 if (push and pull) else 1)
        return per_direction / (float(t.item()) * 1e-3) / 1e9

    out = {"store_one_gpu_gbs": timed(True, False, only_rank0=True), "store_all_gpus_gbs": timed(True, False),
           "load_all_gpus_gbs": timed(False, True), "store_and_load_all_gpus_gbs": timed(True, True),
           "how": f"{nbytes >> 20} MiB per copy with the library's 16-byte copy kernel to / from the next rank's memory, "
                  f"{reps} repetitions, CUDA events, max over ranks; reference figures: 770 GB/s measured peer copy, 900 nominal"}
    torch.cuda.synchronize(dev)
    dist.barrier()
    dp._shared_free(base, peers)
    return out



def measure_pcie(dev, nbytes: int = 1 << 30, reps: int = 5, world: int = 1) -> dict:
    """Plain pinned-memory copy bandwidth of this box: each direction alone and both at once.
    The denominators for the host-buffer paths (PCIe Gen5 x16: 63 GB/s per direction nominal).
    With world > 1 every rank copies at the same time and the slowest rank's rate is reported:
    what the host gives each GPU when all of them move data at once."""
    import torch
    from slideformer_b200.numa import pinned_empty
    h_in = pinned_empty(nbytes, torch.uint8, dev)
    h_out = pinned_empty(nbytes, torch.uint8, dev)
    d_in = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    d_out = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    s1, s2 = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def timed(up: bool, down: bool) -> float:
        torch.cuda.synchronize(dev)
        if world > 1:
            torch.distributed.barrier()
        t0 = time.perf_counter()
        for _ in range(reps):
            if up:
                with torch.cuda.stream(s1):
                    d_in.copy_(h_in, non_blocking=True)
            if down:
                with torch.cuda.stream(s2):
                    h_out.copy_(d_out, non_blocking=True)
        torch.cuda.synchronize(dev)
        return (time.perf_counter() - t0) / reps

    timed(True, True)
    up, down, both = timed(True, False), timed(False, True), timed(True, True)
    if world > 1:
        t = torch.tensor([up, down, both], device=dev, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        up, down, both = (float(x) for x in t)
    return {"h2d_gbs": nbytes / up / 1e9, "d2h_gbs": nbytes / down / 1e9,
            "bidirectional_each_gbs": nbytes / both / 1e9, "nominal_gen5_x16_gbs": 63.0,
            "how": f"{nbytes >> 20} MiB pinned copies, {reps} repetitions, wall clock around a device synchronize"
                   + (f"; all {world} GPUs copying at once, slowest rank" if world > 1 else "")}


# ---------------------------------------------------------------------------------------------
# the CUDA arm
# ---------------------------------------------------------------------------------------------
def main_b200(args):
    import torch
    import torch.distributed as dist
    from slideformer_b200 import LayerAdam, _lib
    from slideformer_b200.host_io import HostGradStepper, pinned_empty

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback for the product path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.load()
    if args.variant >= 0 or args.ctas_per_sm >= 0:
        _lib.check(lib.sf_set_tuning(args.variant, args.ctas_per_sm))
    n = args.n
    K, W = args.steps, max(3, args.warmup)

    sampler = ClockSampler(local)
    sampler.start()
    from slideformer_b200.numa import gpu_numa_cpus
    near = gpu_numa_cpus(dev)
    host_info = {"usable_cpus": cpu_threads(),
                 "pinned_buffers": (f"allocated from the {len(near)} CPUs of the GPU's NUMA node" if near
                                    else "allocated where the process runs (the host exposes no NUMA node for the GPU)")}

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    NG = 3  # rotating gradient buffers: a fresh gradient every step
    extra = {}
    if world == 1:
        p = torch.empty(n, device=dev).normal_(0, 0.02, generator=gen)
        p[-8192:] = 1.0
        m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
        out = torch.empty(n, device=dev, dtype=torch.bfloat16)
        grads = [torch.empty(n, device=dev).normal_(0, 1e-3, generator=gen).to(torch.bfloat16) for _ in range(NG)]
        opt = LayerAdam(**HP)
        group = dict(opt.defaults, step=0)

        def one_step(i):
            group["step"] += 1
            opt.step_chunk(p, grads[i % NG], m, v, group, out)
        hbm_bytes_per_launch = BYTES_PER_PARAM * n
        parallelism = "single GPU, state resident in HBM"
        scaling = "strong"
    else:
        from slideformer_b200.shared_data_parallel import ShardedLayerAdam
        sh = ShardedLayerAdam(numel=n, device=dev, mode=args.dp_mode, **HP)
        sh.params_shard.normal_(0, 0.02, generator=gen)
        for k in range(NG):
            sh.grad_buffer(k).copy_(torch.empty(n, device=dev).normal_(0, 1e-3, generator=gen).to(torch.bfloat16))

        def one_step(i):
            sh.step(i % NG)
        hbm_bytes_per_launch = BYTES_PER_PARAM * sh.shard_numel + 2 * sh.shard_numel * (world - 1 if args.dp_mode != "nccl" else 0)
        parallelism = f"dp{world}: state sharded 1/{world}, {sh.describe()}"
        scaling = "strong"

    # ---- warm-up, then the timed region: K steps, device-timed, max over ranks ----------------
    for i in range(W):
        one_step(i)
    barrier()
    launches0 = lib.sf_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.in_region = True
    e0.record()
    for i in range(K):
        one_step(i)
    e1.record()
    barrier()
    sampler.in_region = False
    launches = lib.sf_launch_count() - launches0
    ms_total = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms_total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_per_step = ms_total / K
    value = n / (ms_per_step * 1e-3) / 1e9

    # ---- per-launch duration of the dominant kernel (roofline numerator) -----------------------
    # at least 0.3 s of launches, so that the clocks are sampled well inside a loaded stretch
    R = int(min(max(K, 50, 300.0 / max(ms_per_step, 1e-3)), 1000))
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(R)]
    if world == 1:
        sampler.in_region = True
        for i in range(R):
            evs[i][0].record()
            one_step(i)
            evs[i][1].record()
        torch.cuda.synchronize()
        sampler.in_region = False
        kern_ms = statistics.mean(a.elapsed_time(b) for a, b in evs)
    else:
        sampler.in_region = True
        kern_ms = sh.time_kernel_only(R)
        sampler.in_region = False
        extra.update(sh.breakdown(50))
        # the same step seen from the data side: every rank contributed one full-layer gradient
        extra["dp_gradient_gparams_per_s"] = world * value
        barrier()
    peak, which = measured_peak()
    achieved = hbm_bytes_per_launch / (kern_ms * 1e-3) / 1e9
    units = n if world == 1 else sh.shard_numel
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": ncu_traffic_bytes(units) if world == 1 else None,
                "peak_source": f"{which} (MEASURED_PEAKS.json hbm_gbs, burst copy)" if which == "measured" else "fallback 6650 GB/s",
                "kernel": "adam_vec4_kernel", "kernel_ms": kern_ms, "launches_timed": R,
                "bytes_per_launch": hbm_bytes_per_launch, "frac_of_nominal_8000": achieved / 8000.0}
    if world > 1 and args.dp_mode == "fused":
        # The fused kernel is bound by NVLink, not HBM: per launch every GPU receives the (N-1)
        # peer gradient slices it pulls plus the (N-1) bf16 slices its peers push into it, and
        # sends as much.  Peak: the 770 GB/s per direction a peer copy reaches on this pool.
        link_bytes = 2 * (world - 1) * sh.shard_numel * 2
        link = link_bytes / (kern_ms * 1e-3) / 1e9
        roofline = {"bound": "nvlink", "achieved": link, "peak": 770.0, "unit": "GB/s", "frac": link / 770.0,
                    "traffic": None, "peak_source": "measured peer copy, 770 GB/s per direction per GPU",
                    "kernel": "adam_push_kernel", "kernel_ms": kern_ms, "launches_timed": R, "bytes_per_launch": link_bytes,
                    "note": "bytes received (= sent) per GPU per launch over NVLink",
                    "hbm": {"achieved": achieved, "peak": peak, "frac": achieved / peak,
                            "bytes_per_launch": hbm_bytes_per_launch}}

    # ---- end to end through the public API with host buffers -----------------------------------
    e2e = None
    if world == 1:
        g_host = [pinned_empty(n, torch.bfloat16, dev) for _ in range(2)]
        for k in range(2):
            g_host[k].copy_(grads[k])
        out_host = pinned_empty(n, torch.bfloat16, dev)
        stepper = HostGradStepper(opt, n, dev, chunk_numel=args.e2e_chunk, min_chunk_numel=args.e2e_min_chunk)
        E = max(3, min(K, 20))
        for i in range(3):
            group["step"] += 1
            stepper.step(p, g_host[i & 1], m, v, out, out_host, group)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        a.record()
        for i in range(E):
            group["step"] += 1
            stepper.step(p, g_host[i & 1], m, v, out, out_host, group, join=False)
        stepper.join()
        b.record()
        torch.cuda.synchronize()
        wall_ms = (time.perf_counter() - t0) * 1e3
        e2e_ms = max(a.elapsed_time(b), wall_ms) / E
        e2e = {"value": n / (e2e_ms * 1e-3) / 1e9, "unit": "Gparams/s", "h2d_bytes_per_step": 2 * n,
               "d2h_bytes_per_step": 2 * n, "ms_per_step": e2e_ms, "steps": E,
               "path": "HostGradStepper: pinned bf16 gradient -> HBM-resident LayerAdam.step_chunk -> pinned bf16 weights, "
                       f"{len(stepper.chunks)} pieces of {args.e2e_min_chunk}..{args.e2e_chunk} elements "
                       "(short at both ends) on three streams"}
        extra["pcie"] = measure_pcie(dev)
        # fully host-resident state (p, m, v and g in pinned host memory) streamed through the GPU
        if args.host_state:
            ph, mh, vh = (pinned_empty(n, torch.float32, dev) for _ in range(3))
            ph.copy_(p)
            mh.zero_()
            vh.zero_()
            hopt = LayerAdam(**HP)
            hg = dict(hopt.defaults, step=0)
            for i in range(4):
                if i == 1:
                    torch.cuda.synchronize()
                    t0 = time.perf_counter()
                hg["step"] += 1
                hopt.step_chunk(ph, g_host[i & 1], mh, vh, hg, out)
            torch.cuda.synchronize()
            hs_ms = (time.perf_counter() - t0) * 1e3 / 3
            extra["e2e_host_state"] = {"value": n / (hs_ms * 1e-3) / 1e9, "unit": "Gparams/s", "ms_per_step": hs_ms,
                                       "h2d_bytes_per_step": 14 * n, "d2h_bytes_per_step": 12 * n,
                                       "h2d_gbs": 14 * n / (hs_ms * 1e-3) / 1e9, "d2h_gbs": 12 * n / (hs_ms * 1e-3) / 1e9,
                                       "path": "sf_adam_update_host: p, m, v, g in pinned host memory, double-buffered chunks"}
            del ph, mh, vh
    else:
        e2e = sh.e2e(K, chunk_numel=args.e2e_chunk, min_chunk_numel=args.e2e_min_chunk)
        extra["pcie"] = measure_pcie(dev, nbytes=1 << 29, world=world)
        e2e["h2d_fraction_of_concurrent_pcie"] = e2e["h2d_gbs_per_gpu"] / extra["pcie"]["h2d_gbs"]
    sampler.stop()

    # ---- the result line: what has been measured so far; the optional sections below add to it ----
    line = {"metric": METRIC, "value": value, "unit": "Gparams/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "parallelism": parallelism,
                       "l2": "inputs (3.05 GB per step) exceed the 126 MB L2; gradient buffer rotates every step",
                       "hyper": {"lr": HP["lr"], "betas": list(HP["betas"]), "eps": HP["eps"], "weight_decay": HP["weight_decay"]}},
            "hbm_gbs": BYTES_PER_PARAM * value, "roofline": roofline, "cpu_baseline": None, "e2e": e2e,
            "gpu_launches": int(launches), "clocks": sampler.summary(), "host": host_info}
    line.update(extra)
    extra = line          # the sections below keep writing into `extra`

    # ---- parity: a few more steps of the very objects that were timed, against the CPU oracle ----
    if not args.no_parity:
        parity = parity_single(dev, p, m, v, out, grads, n) if world == 1 else parity_sharded(sh, world, rank, dev)
        if parity["mismatches"]:
            raise SystemExit(f"parity check failed: {parity}")
        extra["parity"] = parity

    if world == 1 and rank == 0 and not args.no_cpu_baseline:
        r = run_cpu_arm(n, 8, 2, budget_s=20.0)
        line["cpu_baseline"] = {"value": r["value"], "unit": "Gparams/s", "cores": r["cores"], "kind": r["kind"],
                                "sample": r["sample"], "ms_per_step": r["ms_per_step"], "bf16_cast_ms": r["bf16_cast_ms"]}

    # Everything from here on is additional reporting.  If one of these sections ever stalls (a
    # collective that a peer never joins), the line measured so far is still printed: a timer on
    # every rank ends the process at the deadline, rank 0 after emitting the line.
    section = ["sweep"]
    done = threading.Event()
    emit_lock = threading.Lock()

    def finish(truncated=None):
        with emit_lock:
            if done.is_set():
                return
            done.set()
            if truncated:
                line["truncated"] = f"deadline of {args.deadline:.0f} s reached during the '{truncated}' section"
            if rank == 0:
                emit(json.dumps(line))

    def on_deadline():
        finish(section[0])
        os._exit(0)

    timer = threading.Timer(max(1.0, args.deadline - (time.perf_counter() - T_START)), on_deadline)
    timer.daemon = True
    timer.start()

    # ---- the size sweep (kernel alone at N = 1; kernel and whole step when sharded) --------------
    if not args.no_sweep:
        main_entry = {"n": n, "ms": ms_per_step, "kernel_ms": kern_ms, "gparams_per_s": value,
                      "frac": roofline["frac"], "launches": K, "l2": "inputs exceed L2"}
        if world == 1:
            main_entry["hbm_gbs"] = BYTES_PER_PARAM * value
            extra["sweep"] = sweep_single(dev, peak, main_entry)
        else:
            main_entry["nvlink_gbs_per_direction"] = roofline.get("achieved")
            extra["sweep"] = sweep_sharded(dev, world, args.dp_mode, main_entry)
    section[0] = "nvlink"
    if world > 1 and not args.no_nvlink:
        extra["nvlink"] = measure_nvlink(sh.dp, dev)
        if roofline.get("bound") == "nvlink":
            both = extra["nvlink"]["store_and_load_all_gpus_gbs"]
            roofline["frac_of_measured_bidirectional_copy"] = roofline["achieved"] / both
    section[0] = "fast_mode"
    if world > 1 and args.dp_mode == "fused" and not args.no_fast_mode:
        extra["fast_mode"] = fast_mode_nvls(sh, dev, world, n)

    # ---- fine-tune tokens/s with the same kernel inside the layer-sliding engine ------------------
    section[0] = "finetune"
    if args.finetune != "none":
        import gc
        from slideformer_b200.finetune_bench import run_finetune
        if world == 1:
            del p, m, v, out, grads, g_host, out_host, stepper, opt
        else:
            sh.close()
            del sh
        gc.collect()
        torch.cuda.empty_cache()
        # (model, batch per GPU, seq, timed steps, warm-up, state placement, window mode + meta build, HBM budget)
        jobs = [("gpt2-small", 8, 1024, 20, 5, "hbm", False, None), ("llama3.1-8b", 8, 1024, 4, 2, "hbm", False, None)]
        if world == 1:
            # the configuration as the benchmark list words it: host-pinned optimizer state ...
            jobs.append(("llama3.1-8b", 8, 1024, 2, 1, "host", False, None))
            # ... and the middle ground: state in HBM while a 64 GB budget lasts, the rest streamed
            jobs.append(("llama3.1-8b", 8, 1024, 2, 1, "auto", False, 64.0))
        if world == 8:
            # Llama-3.1-70B: state sharded 1/8, bf16 weights kept as slices and gathered per layer
            jobs.append(("llama3.1-70b", 4, 2048, 2, 1, "hbm", True, None))
        line["finetune"] = []
        for name, fbatch, fseq, fsteps, fwarm, state_dev, window, budget in jobs:
            section[0] = f"finetune {name} ({state_dev})"
            dp = None
            if world > 1:
                from slideformer_b200.shared_data_parallel import SharedDataParallel
                dp = SharedDataParallel(dtype=torch.bfloat16, exchange_slots=2)
            line["finetune"].append(run_finetune(name, fbatch, fseq, fsteps, fwarm, dev, world, rank, dp, state_device=state_dev,
                                                 weight_window=window, meta=window, hbm_state_budget_gb=budget))
            if dp is not None:
                dp.close()

    timer.cancel()
    finish()
    if world > 1:
        dist.destroy_process_group()
    return 0


def main():
    # Libraries (NCCL's version banner, for one) print to stdout; the contract is ONE JSON line
    # there, so everything but the final line is sent to stderr at the file-descriptor level.
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--n", type=int, default=N_LAYER, help="flat layer size (parity and sweep runs only)")
    ap.add_argument("--dp-mode", default="fused", choices=["fused", "fused_ag", "nccl", "nvls"])
    ap.add_argument("--e2e-chunk", type=int, default=16 * 1024 * 1024)
    ap.add_argument("--e2e-min-chunk", type=int, default=4 * 1024 * 1024)
    ap.add_argument("--host-state", action="store_true", default=True)
    ap.add_argument("--no-host-state", dest="host_state", action="store_false")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--deadline", type=float, default=780.0,
                    help="seconds after start at which the line measured so far is printed and the run ends, should an "
                         "additional-reporting section (sweep, NVLink yardstick, NVLS variant, fine-tune) still be running")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle check of extra steps after the timed region")
    ap.add_argument("--no-sweep", action="store_true", help="skip the 1M / 16M / 218M / 1B size sweep")
    ap.add_argument("--no-nvlink", action="store_true", help="N > 1: skip the bare-copy NVLink measurement")
    ap.add_argument("--no-fast-mode", action="store_true",
                    help="N > 1: skip the NVLS (in-switch reduction) variant that is reported beside the exact kernel")
    ap.add_argument("--variant", type=int, default=-1,
                    help="access pattern of the kernel (sf_set_tuning): 0 default caching, 1 streaming hints, 2 256-bit")
    ap.add_argument("--ctas-per-sm", type=int, default=-1, help="0 = one tile per CTA, k > 0 = persistent grid")
    ap.add_argument("--finetune", default="all", choices=["none", "all"],
                    help="also report fine-tune tokens/s through the engine: GPT-2 small and Llama-3.1-8B (batch 8 x 1024 "
                         "per GPU), Llama-3.1-8B with host-pinned state at N=1, Llama-3.1-70B (batch 4 x 2048 per GPU) at N=8")
    args = ap.parse_args()
    if args.impl == "reference":
        return main_reference(args)
    return main_b200(args)


if __name__ == "__main__":
    sys.exit(main())
