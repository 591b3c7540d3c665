"""Benchmark of the fused multi-feature embedding-bag forward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg3]

One "step" = one fused forward over one synthetic batch of the workload
(default: the heavy-tailed 200-feature fp16 configuration, batch 16384, about
120 GB of tables replicated on every GPU; ranks split the batch stream, no
collective on the data path).  Rank 0 prints one JSON line:

  value     whole-job samples/s with the batch already resident in HBM
  e2e       the same through the host-buffer call (H2D of indices/offsets and D2H
            of the pooled output inside the timed region)
  roofline  algorithmic bytes (gathered rows + indices + offsets) of one launch
            divided by the fused kernel's mean CUDA-event duration, against the
            measured HBM copy bandwidth in MEASURED_PEAKS.json
  cpu_baseline  torch.nn.functional.embedding_bag(mode='sum') on the host cores
            on a bounded sample of the same batch (reported only)

`--impl reference` times that CPU path alone (the reference has no CPU
implementation of its own; the benchmark definition names torch EmbeddingBag
on the host cores as its CPU path).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np

METRIC = "fused_embedding_bag_samples_per_s"
UNIT = "samples/s"
WORKLOADS = {"cfg1": 1, "cfg2": 2, "cfg3": 3, "cfg4": 4, "cfg5": 5}


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=100)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", choices=["ours", "reference"], default="ours")
    p.add_argument("--workload", choices=sorted(WORKLOADS), default="cfg3")
    p.add_argument("--row-scale", type=float, default=1.0, help="shrink every table (debugging only; the line says so)")
    p.add_argument("--batch", type=int, default=0, help="override the batch size (debugging only)")
    p.add_argument("--batches", type=int, default=4, help="distinct batches rotated through the steps")
    p.add_argument("--schedules", type=str, default="", help="JSON file written by the tuner (default: tuned/<workload>.json if present)")
    p.add_argument("--occupancy", type=int, default=0)
    p.add_argument("--overlap", type=int, default=-1,
                   help="CTAs per SM of the fused kernel while the warp-per-bag kernel runs beside it (0 = one after "
                        "the other; default: the tuned file's value, else 0)")
    p.add_argument("--kind", type=str, default="", help="force one schedule kind for every feature (debugging)")
    p.add_argument("--unroll", type=int, default=0)
    p.add_argument("--cpu-seconds", type=float, default=12.0, help="CPU baseline budget")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--chunks", type=int, default=4, help="batch chunks of the sharded path (exchange/pooling overlap)")
    p.add_argument("--tune", action="store_true", help="run the two-stage tuner on the first batch before timing (untimed)")
    p.add_argument("--emulate-world", type=int, default=0,
                   help="sharded workloads on ONE GPU: build only rank --emulate-rank's shard of a sharding over this "
                        "many ranks and time its pooling alone (no exchange); for profiling a shard")
    p.add_argument("--emulate-rank", type=int, default=0)
    p.add_argument("--compare-batch-order", action="store_true",
                   help="sharded path, peer exchange: also time the steps with tiles walked in batch order "
                        "(destination interleave off) and report that time beside the headline")
    p.add_argument("--probe-exchange", action="store_true",
                   help="sharded path, peer exchange: also time the steps on a batch of empty bags, i.e. the same "
                        "stores to the same addresses with nothing gathered (the exchange alone)")
    p.add_argument("--exchange", choices=["peer", "nccl"], default="peer",
                   help="sharded path: fused peer-memory stores, or pool + NCCL all-to-all + placement")
    return p.parse_args()


# ---------------------------------------------------------------------------
# clocks (read-only NVML polling during the timed regions)
# ---------------------------------------------------------------------------
class ClockSampler:
    REASONS = {
        0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
        0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
        0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting",
    }

    def __init__(self, index: int):
        self.samples, self.reason_bits = [], 0
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                try:
                    bits = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                except Exception:
                    bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                self.reason_bits |= int(bits) & ~0x1
            except Exception:
                pass
            self._stop.wait(0.02)

    def start(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["nvml_unavailable"]}
        reasons = [name for bit, name in self.REASONS.items() if self.reason_bits & bit]
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz, "reasons": reasons,
                "samples": len(self.samples)}


# ---------------------------------------------------------------------------
# CPU path (reported baseline and the reference arm)
# ---------------------------------------------------------------------------
def cpu_sample(cfg, values, offsets, bags: int):
    """First `bags` bags of every feature with tables compacted to the rows they touch
    (the full tables exist only on the GPU); returns (tables, values, offsets) for the oracle."""
    from recflex_b200 import synth

    tabs, vals, offs = [], [], []
    for fs, v, o in zip(cfg.features, values, offsets):
        o = np.asarray(o[: bags + 1], dtype=np.int64)
        v = np.asarray(v[: o[-1]], dtype=np.int64)
        uniq, inv = np.unique(v, return_inverse=True)
        if len(uniq) == 0:
            uniq = np.zeros(1, dtype=np.int64)
        tabs.append(synth.synth_rows(fs.seed, uniq, fs.dim, fs.dtype))
        vals.append(inv.astype(np.int64))
        offs.append(o)
    return tabs, vals, offs


def time_cpu(cfg, values, offsets, seconds: float, steps: int = 0, warmup: int = 1):
    import torch

    from oracle import oracle

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    bags = min(1024, len(offsets[0]) - 1)
    tabs, vals, offs = cpu_sample(cfg, values, offsets, bags)
    tabs_t = [torch.from_numpy(t).float() for t in tabs]
    vals_t = [torch.from_numpy(v) for v in vals]
    offs_t = [torch.from_numpy(o) for o in offs]
    for _ in range(max(1, warmup)):
        oracle.pool_torch(tabs_t, vals_t, offs_t)
    t0 = time.perf_counter()
    reps = 0
    while True:
        oracle.pool_torch(tabs_t, vals_t, offs_t)
        reps += 1
        el = time.perf_counter() - t0
        if (steps and reps >= steps) or (not steps and el >= seconds):
            break
        if steps and el > 240:
            break
    return {
        "value": reps * bags / el,
        "unit": UNIT,
        "cores": cores,
        "kind": "port",
        "sample": f"torch.nn.functional.embedding_bag(mode='sum') per feature, fp32, {cores} threads; first {bags} bags of "
                  f"each of {len(cfg.features)} features of one batch, tables compacted to the rows touched; "
                  f"{reps} passes in {el:.1f} s",
        "ms_per_step": el / reps * 1e3,
        "reps": reps,
    }


def run_reference(args):
    """CPU arm: rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from recflex_b200 import synth

    cfg = synth.make_config(WORKLOADS[args.workload], row_scale=args.row_scale, batch=args.batch or None)
    values, offsets = synth.gen_batch(cfg, seed=0)
    res = time_cpu(cfg, values, offsets, args.cpu_seconds, steps=args.steps, warmup=args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": res["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": res["reps"], "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(cfg, args),
        "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": res["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(cfg, args):
    return {
        "workload": cfg.name,
        "features": len(cfg.features),
        "batch_per_gpu": cfg.batch,
        "table_dtype": cfg.features[0].dtype,
        "table_gb_per_gpu": round(cfg.table_bytes / 1e9, 2),
        "output_units": cfg.output_units,
        "partitioning": "tables replicated on every GPU, each rank pools its own batches (no data-path collective)",
        "l2": f"inputs larger than L2: {cfg.table_bytes / 1e9:.0f} GB of tables, {args.batches} distinct batches rotated",
        "row_scale": args.row_scale,
    }


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist

    from recflex_b200 import _lib, synth
    from recflex_b200.rec_modules import FeatEmbed, Schedule

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the fused forward has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    cfg = synth.make_config(WORKLOADS[args.workload], row_scale=args.row_scale, batch=args.batch or None)
    B, F = cfg.batch, len(cfg.features)
    tables = synth.make_tables_device(cfg, dev)
    torch.cuda.synchronize()
    mod = FeatEmbed(dev, embed_tables=tables)

    sched_path = args.schedules or os.path.join(ROOT, "recflex_b200", "tuned", f"{args.workload}.json")
    sched_note = "library defaults"
    if args.kind:
        mod.set_schedules([Schedule(args.kind, args.unroll) for _ in range(F)], occupancy=args.occupancy)
        sched_note = f"forced {args.kind} unroll {args.unroll}"
    elif os.path.exists(sched_path):
        with open(sched_path) as f:
            tuned = json.load(f)
        if len(tuned["schedules"]) == F:
            mod.set_schedules([Schedule.from_json(s) for s in tuned["schedules"]],
                              occupancy=args.occupancy or tuned.get("occupancy", 0))
            sched_note = f"tuned ({os.path.relpath(sched_path, ROOT)})"
    elif args.occupancy:
        mod.set_schedules(None, occupancy=args.occupancy)
    _, occupancy = mod.get_schedules()
    overlap = args.overlap
    if overlap < 0:
        overlap = int(tuned.get("overlap", 0)) if sched_note.startswith("tuned (") else 0
    if overlap:
        mod.set_kernel_overlap(overlap)
        sched_note += f"; warp-per-bag kernel beside the fused kernel ({overlap} CTAs/SM)"

    # distinct batches, different on every rank; kept packed on the host (pinned) and on the device
    host_v, host_o, dev_v, dev_o, alg_bytes = [], [], [], [], []
    first = None
    for i in range(args.batches):
        values, offsets = synth.gen_batch(cfg, seed=1000 * rank + i)
        if first is None:
            first = (values, offsets)
        alg_bytes.append(synth.algorithmic_bytes(cfg, offsets, 4))
        pv, po = synth.pack_batch(values, offsets)
        hv, ho = torch.from_numpy(pv).pin_memory(), torch.from_numpy(po).pin_memory()
        host_v.append(hv)
        host_o.append(ho)
        dev_v.append(hv.to(dev))
        dev_o.append(ho.to(dev))
    out = torch.empty((B, cfg.output_units), dtype=torch.float32, device=dev)
    host_out = torch.empty((B, cfg.output_units), dtype=torch.float32).pin_memory()
    nb = args.batches
    if args.tune:
        from recflex_b200.tuning import TuneConfig, Tuner

        tb = [([torch.from_numpy(v).to(dev) for v in first[0]], [torch.from_numpy(o).to(dev) for o in first[1]])]
        res = Tuner(mod, tb, TuneConfig()).tune()
        sched_note = f"tuned before timing (occupancy {res.occupancy})"
        overlap = res.overlap
        if overlap:
            sched_note += f"; warp-per-bag kernel beside the fused kernel ({overlap} CTAs/SM)"
        if args.schedules:
            res.save(args.schedules, workload=cfg.name)
        del tb
        _, occupancy = mod.get_schedules()

    per_step_launches = 2 + (1 if any(s.kind == _lib.EB_SCHED_WARP for s in mod.get_schedules()[0]) else 0)
    for i in range(max(3, args.warmup)):
        mod.forward_packed(dev_v[i % nb], dev_o[i % nb], out=out)
    mod.check_status()

    sampler = ClockSampler(local_rank)
    # ---- timed region A: inputs resident in HBM ----
    mod.kernel_timing(True)
    K = args.steps
    barrier()
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(K):
        mod.forward_packed(dev_v[i % nb], dev_o[i % nb], out=out)
    ev1.record()
    barrier()
    t_dev = ev0.elapsed_time(ev1) * 1e-3
    ktimes = []
    # the event ring holds 256 launches; longer runs time the first 256
    ktimes = mod.kernel_times()
    mod.kernel_timing(False)

    # ---- timed region B: host buffers in, host result out ----
    # Two handles over the same tables alternate on two streams, so that step k + 1's upload overlaps step k's
    # download (PCIe is full duplex); each call is still upload -> bind + fused kernel -> download of its result.
    t_e2e = None
    if not args.no_e2e:
        mod_b = FeatEmbed(dev, embed_tables=tables)
        scheds, occ_b = mod.get_schedules()
        mod_b.set_schedules(scheds, occupancy=occ_b)
        if overlap:
            mod_b.set_kernel_overlap(overlap)
        lanes = [(mod, torch.cuda.Stream(device=dev), host_out),
                 (mod_b, torch.cuda.Stream(device=dev), torch.empty_like(host_out).pin_memory())]

        def e2e_steps(n):
            main = torch.cuda.current_stream(dev)
            for _, st, _ in lanes:
                st.wait_stream(main)
            for i in range(n):
                m, st, ho = lanes[i % 2]
                with torch.cuda.stream(st):
                    m.forward_host(host_v[i % nb], host_o[i % nb], out=ho)
            for _, st, _ in lanes:
                main.wait_stream(st)

        e2e_steps(2)
        barrier()
        ev2, ev3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev2.record()
        e2e_steps(K)
        ev3.record()
        barrier()
        t_e2e = ev2.elapsed_time(ev3) * 1e-3
    sampler.stop()

    if world > 1:
        t = torch.tensor([t_dev, t_e2e or 0.0], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        t_dev, t_e2e_max = float(t[0]), float(t[1])
        t_e2e = t_e2e_max if t_e2e is not None else None

    if rank == 0:
        peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
        if os.path.exists(peaks_path):
            with open(peaks_path) as f:
                peak, peak_src = float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        else:
            peak, peak_src = 6650.0, "fallback"
        traffic = None  # dram__bytes_read + dram__bytes_write of one full-size launch, from the committed ncu summary
        prof = os.path.join(ROOT, "profiles", f"eb_fused_kernel_{args.workload}_full_size.md")
        if os.path.exists(prof) and args.row_scale == 1.0 and not args.batch:
            import re

            with open(prof) as f:
                m = re.search(r"dram_bytes_per_launch:\s*(\d+)", f.read())
            traffic = int(m.group(1)) if m else None
        k_ms = statistics.mean(ktimes) if ktimes else None
        mean_bytes = statistics.mean(alg_bytes[i % nb] for i in range(min(K, 256)))
        achieved = mean_bytes / (k_ms * 1e-3) / 1e9 if k_ms else None
        h2d = int(host_v[0].numel() * 4 + host_o[0].numel() * 4)
        d2h = int(B * cfg.output_units * 4)
        line = {
            "metric": METRIC, "value": world * K * B / t_dev, "unit": UNIT, "n_gpus": world, "steps": K,
            "warmup": max(3, args.warmup), "ms_per_step": t_dev / K * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {**workload_config(cfg, args), "schedules": sched_note, "occupancy": occupancy,
                       "index_dtype": "int32"},
            "roofline": {
                "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak if achieved else None, "traffic": traffic,
                "kernel": "eb_fused_kernel", "kernel_ms": k_ms, "algorithmic_bytes_per_launch": mean_bytes,
                "peak_source": peak_src,
            },
            "e2e": {"value": world * K * B / t_e2e if t_e2e else None, "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": t_e2e / K * 1e3 if t_e2e else None},
            # binding kernel + fused kernel per step, + the warp-per-bag kernel when a feature is on that schedule
            "gpu_launches": per_step_launches * K + (per_step_launches * K if t_e2e else 0),
            "clocks": sampler.summary(),
        }
        if world == 1 and not args.no_cpu_baseline:
            res = time_cpu(cfg, first[0], first[1], args.cpu_seconds)
            line["cpu_baseline"] = {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def plan_cfg_shards(cfg, world, cap):
    """Owner rank per table + summary for the sharded workload: balances what every rank gathers AND what it sends
    (one-hot features send twice the bytes they gather from an fp16 table), with table bytes kept within 15 % of an
    even split where that is feasible."""
    from recflex_b200 import synth
    from recflex_b200.sharding import plan_shards, shard_summary

    table_bytes = [fs.table_bytes for fs in cfg.features]
    traffic = synth.expected_traffic(cfg)
    sent = [cfg.batch * fs.dim * 4 * (world - 1) / world for fs in cfg.features]
    try:
        owner = plan_shards(table_bytes, traffic, world, min(cap, int(1.15 * sum(table_bytes) / world)), exchange=sent)
    except ValueError:
        owner = plan_shards(table_bytes, traffic, world, cap, exchange=sent)
    return owner, shard_summary(owner, table_bytes, traffic, world, exchange=sent)


def run_shard_emulation(args):
    """One rank's shard of cfg4 on a single GPU: pooling only, for profiling (not a benchmark line of the job)."""
    import torch

    from recflex_b200 import synth
    from recflex_b200.rec_modules import FeatEmbed
    from recflex_b200.sharding import plan_shards

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    cfg = synth.make_config(WORKLOADS[args.workload], row_scale=args.row_scale, batch=args.batch or None)
    W, R, B = args.emulate_world, args.emulate_rank, cfg.batch
    owner, _ = plan_cfg_shards(cfg, W, int(torch.cuda.mem_get_info(dev)[1] * 0.88))
    local = [f for f, r in enumerate(owner) if r == R]
    mod = FeatEmbed(dev, embed_tables=synth.make_tables_device(cfg, dev, features=local))
    mod.set_schedules(None, occupancy=args.occupancy or 6)
    batches, alg = [], []
    for i in range(args.batches):
        vs, os_, nbytes = [], [], 0
        for f in local:
            v, o = synth.gen_feature_batch(cfg.features[f], B, seed=i)
            nbytes += int(o[-1]) * cfg.features[f].row_bytes + int(o[-1]) * 4 + len(o) * 4
            vs.append(torch.from_numpy(v.astype(np.int32)).to(dev))
            os_.append(torch.from_numpy(o.astype(np.int32)).to(dev))
        batches.append((vs, os_))
        alg.append(nbytes)
    if args.tune:
        from recflex_b200.tuning import TuneConfig, Tuner

        Tuner(mod, [batches[0]], TuneConfig(occupancies=(3, 4, 5, 6, 8), reps=1, global_reps=2)).tune()
    out = torch.empty((B, mod.output_units), dtype=torch.float32, device=dev)
    for i in range(max(3, args.warmup)):
        mod(*batches[i % len(batches)], out=out)
    mod.kernel_timing(True)
    for i in range(args.steps):
        mod(*batches[i % len(batches)], out=out)
    kt = mod.kernel_times()
    k_ms = statistics.mean(kt)
    scheds, occ = mod.get_schedules()
    print(json.dumps({"emulated_rank": R, "of": W, "workload": cfg.name, "local_features": len(local),
                      "table_gb": round(sum(cfg.features[f].table_bytes for f in local) / 1e9, 1),
                      "kernel_ms": k_ms, "algorithmic_bytes_per_launch": statistics.mean(alg),
                      "algorithmic_gbs": statistics.mean(alg) / (k_ms * 1e-3) / 1e9, "occupancy": occ,
                      "note": "pooling of one shard only; no exchange"}), flush=True)


def run_sharded(args):
    """cfg4: tables sharded table-wise over the ranks, pooled outputs exchanged with an all-to-all."""
    import torch
    import torch.distributed as dist

    from recflex_b200 import synth
    from recflex_b200.sharding import ShardedFeatEmbed, plan_shards, shard_summary

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the fused forward has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    dist.init_process_group("nccl", device_id=dev, rank=rank, world_size=world)

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    cfg = synth.make_config(WORKLOADS[args.workload], row_scale=args.row_scale, batch=args.batch or None)
    B, F = cfg.batch, len(cfg.features)
    table_bytes = [fs.table_bytes for fs in cfg.features]
    traffic = synth.expected_traffic(cfg)
    free_b, total_b = torch.cuda.mem_get_info(dev)
    cap = int(total_b * 0.88)
    if sum(table_bytes) > cap * world:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "unavailable": f"{cfg.name}: {sum(table_bytes) / 1e9:.0f} GB of tables do "
                              f"not fit {world} GPU(s) of {total_b / 1e9:.0f} GB", "n_gpus": world}), flush=True)
        dist.destroy_process_group()
        return
    dims = [fs.dim for fs in cfg.features]
    owner, summ = plan_cfg_shards(cfg, world, cap)
    local = [f for f, r in enumerate(owner) if r == rank]
    tables = synth.make_tables_device(cfg, dev, features=local)
    mod = ShardedFeatEmbed(rank, world, owner, dims, local_tables=tables, device=dev, chunks=args.chunks,
                           exchange=args.exchange)
    mod.set_batch_for_empty_rank(B)
    if mod.local is not None:
        mod.local.set_schedules(None, occupancy=args.occupancy or 6)
    tuned_note = "library defaults"

    nb = args.batches
    host, devb, alg = [], [], []
    for i in range(nb):
        hv, ho, bytes_i = [], [], 0
        for f in local:
            v, o = synth.gen_feature_batch(cfg.features[f], B, seed=i)
            bytes_i += int(o[-1]) * cfg.features[f].row_bytes + int(o[-1]) * 4 + len(o) * 4
            hv.append(torch.from_numpy(v.astype(np.int32)).pin_memory())
            ho.append(torch.from_numpy(o.astype(np.int32)).pin_memory())
        host.append((hv, ho))
        devb.append(([t.to(dev) for t in hv], [t.to(dev) for t in ho]))
        alg.append(bytes_i)
    if args.tune and mod.local is not None:
        from recflex_b200.tuning import TuneConfig, Tuner

        res = Tuner(mod.local, [devb[0]], TuneConfig(occupancies=(4, 5, 6, 8), reps=1, global_reps=2)).tune()
        tuned_note = f"tuned per rank before timing (rank 0: occupancy {res.occupancy})"
    host_out = torch.empty((B // world, cfg.output_units), dtype=torch.float32).pin_memory()
    if args.exchange == "peer":
        run_step = lambda v, o: mod(v, o)
    else:
        out_buf = torch.empty((B // world, cfg.output_units), dtype=torch.float32, device=dev)
        run_step = lambda v, o: mod(v, o, out=out_buf)
    for i in range(max(3, args.warmup)):
        out = run_step(*devb[i % nb])
    if mod.local is not None:
        mod.local.check_status()

    sampler = ClockSampler(local_rank)
    K = args.steps
    if mod.local is not None:
        mod.local.kernel_timing(True)
    barrier()
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(K):
        run_step(*devb[i % nb])
    ev1.record()
    barrier()
    t_dev = ev0.elapsed_time(ev1) * 1e-3
    ktimes = mod.local.kernel_times() if mod.local is not None else []
    if mod.local is not None:
        mod.local.kernel_timing(False)

    t_plain = 0.0
    if args.compare_batch_order and args.exchange == "peer":
        if mod.local is not None:
            mod.local.set_peer_interleave(False)
        for i in range(3):
            run_step(*devb[i % nb])
        barrier()
        ev4, ev5 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev4.record()
        for i in range(K):
            run_step(*devb[i % nb])
        ev5.record()
        barrier()
        t_plain = ev4.elapsed_time(ev5) * 1e-3
        if mod.local is not None:
            mod.local.set_peer_interleave(True)

    t_probe = 0.0
    if args.probe_exchange and args.exchange == "peer":
        ev = [torch.zeros(1, dtype=torch.int32, device=dev) for _ in local]
        eo = [torch.zeros(B + 1, dtype=torch.int32, device=dev) for _ in local]
        for i in range(3):
            run_step(ev, eo)
        barrier()
        ev6, ev7 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev6.record()
        for i in range(K):
            run_step(ev, eo)
        ev7.record()
        barrier()
        t_probe = ev6.elapsed_time(ev7) * 1e-3

    t_e2e = None
    if not args.no_e2e:
        def e2e_step(i):
            hv, ho = host[i % nb]
            dv = [t.to(dev, non_blocking=True) for t in hv]
            do = [t.to(dev, non_blocking=True) for t in ho]
            host_out.copy_(run_step(dv, do), non_blocking=True)

        e2e_step(0)
        barrier()
        ev2, ev3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev2.record()
        for i in range(K):
            e2e_step(i)
        ev3.record()
        barrier()
        t_e2e = ev2.elapsed_time(ev3) * 1e-3
    sampler.stop()

    launches_per_step = 1 if args.exchange == "peer" else args.chunks
    k_sum = sum(ktimes) / max(1, min(K, 256 // launches_per_step)) if ktimes else 0.0  # pooled-kernel ms per step, this rank
    stats = torch.tensor([t_dev, t_e2e or 0.0, k_sum, float(sum(alg) / len(alg)), t_plain, t_probe], dtype=torch.float64,
                         device=dev)
    mx = stats.clone()
    dist.all_reduce(mx, op=dist.ReduceOp.MAX)
    sm = stats.clone()
    dist.all_reduce(sm, op=dist.ReduceOp.SUM)
    if rank == 0:
        peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
        peak = float(json.load(open(peaks_path))["hbm_gbs"]) if os.path.exists(peaks_path) else 6650.0
        t_dev, t_e2e_m, k_max, _, t_plain_m, t_probe_m = [float(x) for x in mx]
        total_alg = float(sm[3])
        h2d = sum(t.numel() * 4 for t in host[0][0]) + sum(t.numel() * 4 for t in host[0][1])
        exch = max(summ["exchange_per_rank"])  # bytes the busiest rank sends per step
        achieved = (total_alg / world) / (k_max * 1e-3) / 1e9 if k_max else None
        line = {
            "metric": METRIC, "value": K * B / t_dev, "unit": UNIT, "n_gpus": world, "steps": K,
            "warmup": max(3, args.warmup), "ms_per_step": t_dev / K * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": cfg.name, "features": F, "global_batch": B, "table_dtype": cfg.features[0].dtype,
                       "table_gb_total": round(cfg.table_bytes / 1e9, 1), "output_units": cfg.output_units,
                       "partitioning": f"table-wise shards over {world} ranks (LPT planner, gather traffic imbalance "
                                       f"{summ['traffic_imbalance']:.3f}, sent bytes imbalance "
                                       f"{summ['exchange_imbalance']:.3f}); exchange: " +
                                       ("pooled rows stored by the fused kernel into the destination rank's output "
                                        "over NVLink peer memory, one-element all-reduce as the barrier"
                                        if args.exchange == "peer" else
                                        f"NCCL all-to-all of pooled fp32 rows in {args.chunks} chunks + placement kernel"),
                       "exchange_bytes_sent_per_rank_per_step": int(exch), "row_scale": args.row_scale,
                       "l2": f"inputs larger than L2: {max(summ['bytes_per_rank']) / 1e9:.0f} GB of tables per rank, "
                             f"{nb} distinct batches rotated", "schedules": tuned_note},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak if achieved else None, "traffic": None, "kernel": "eb_fused_kernel",
                         "kernel_ms": k_max, "algorithmic_bytes_per_launch": total_alg / world,
                         "note": "slowest rank's pooled-kernel time per step (sum over chunks) against the mean "
                                 "per-rank algorithmic bytes"},
            "e2e": {"value": K * B / t_e2e_m if t_e2e_m else None, "unit": UNIT, "h2d_bytes_per_step": int(h2d),
                    "d2h_bytes_per_step": int(B // world * cfg.output_units * 4),
                    "ms_per_step": t_e2e_m / K * 1e3 if t_e2e_m else None},
            "gpu_launches": K * (2 if args.exchange == "peer" else args.chunks * 3),
            "clocks": sampler.summary(),
        }
        if t_plain_m:
            line["config"]["batch_order_ms_per_step"] = t_plain_m / K * 1e3
        if t_probe_m:
            line["config"]["exchange_alone_ms_per_step"] = t_probe_m / K * 1e3
            line["config"]["exchange_alone_gbs_per_rank"] = exch / (t_probe_m / K) / 1e9
        print(json.dumps(line), flush=True)
    dist.barrier()
    if args.exchange == "peer":
        mod.close()
    dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "cfg4" and args.emulate_world:
        run_shard_emulation(args)
    elif args.workload == "cfg4":
        run_sharded(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
