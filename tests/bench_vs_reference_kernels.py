"""Times the reference's own device templates on a B200 beside this library's fused kernel (manual run).

    python tests/bench_vs_reference_kernels.py --workload cfg2 [--reps 20]

The reference's generated FusedKnl is not built here (generated code + libtorch); what runs is its per-feature
device code (ws::SparseSegmentReduce, obms::SparseSegmentReduce, onehot::GatherSegments) from
oracle/_ref/libref_kernels.so, one launch per feature.  Two figures are reported for it: the sum of each
feature's best (ws or obms) kernel time launched alone, and the wall time (CUDA events) of all features' best
kernels launched over 16 streams so that they can overlap the way the features of one fused kernel do.  Both use
fixed, reasonable template parameters (see oracle/ref_kernels.cu), not the reference's tuner.  The reference
supports fp32 tables and int32 indices only, so this covers cfg1, cfg2 and cfg5.
"""
import argparse
import ctypes as C
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch

from recflex_b200 import synth
from recflex_b200.rec_modules import FeatEmbed, Schedule


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="cfg2", choices=["cfg1", "cfg2", "cfg5"])
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--per-feature", action="store_true", help="also time every feature alone in this library")
    ap.add_argument("--only-feature", type=int, default=-1, help="run just this feature, alone, with both sides (for ncu)")
    ap.add_argument("--kind", default="stream")
    ap.add_argument("--unroll", type=int, default=4)
    ap.add_argument("--occupancy", type=int, default=8)
    args = ap.parse_args()
    ref = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libref_kernels.so"))
    ref.ref_pool_feature.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                     C.c_void_p]
    ref.ref_onehot_feature.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
    dev = torch.device("cuda", 0)
    cfg = synth.make_config(int(args.workload[3:]))
    tables = synth.make_tables_device(cfg, dev)
    values, offsets = synth.gen_batch(cfg, seed=0)
    dv = [torch.from_numpy(v).to(dev) for v in values]
    do = [torch.from_numpy(o).to(dev) for o in offsets]
    B = cfg.batch
    outs = [torch.empty((B, fs.dim), dtype=torch.float32, device=dev) for fs in cfg.features]

    def launch(f, kind, stream):
        t, v, o, out = tables[f], dv[f], do[f], outs[f]
        sp = C.c_void_p(stream.cuda_stream)
        if kind == "onehot":
            rc = ref.ref_onehot_feature(t.shape[1], t.data_ptr(), v.data_ptr(), out.data_ptr(), v.numel(), sp)
        else:
            rc = ref.ref_pool_feature(0 if kind == "ws" else 1, t.shape[1], t.data_ptr(), v.data_ptr(), o.data_ptr(),
                                      out.data_ptr(), v.numel(), B, sp)
        assert rc == 0, (f, kind, rc)

    def time_alone(f, kind):
        st = torch.cuda.current_stream()
        for _ in range(3):
            launch(f, kind, st)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.reps):
            launch(f, kind, st)
        e1.record()
        e1.synchronize()
        return e0.elapsed_time(e1) / args.reps

    if args.only_feature >= 0:
        f = args.only_feature
        fs = cfg.features[f]
        for k in (["onehot"] if fs.length == "onehot" else ["ws", "obms"]):
            print(k, "ref_us", round(time_alone(f, k) * 1e3, 1))
        one = FeatEmbed(dev, embed_tables=[tables[f]])
        one.set_schedules([Schedule(args.kind, args.unroll)], occupancy=args.occupancy)
        o1 = torch.empty((B, fs.dim), dtype=torch.float32, device=dev)
        for _ in range(3):
            one([dv[f]], [do[f]], out=o1)
        one.kernel_timing(True)
        for _ in range(5):
            one([dv[f]], [do[f]], out=o1)
        kt = one.kernel_times()
        print(args.kind, args.unroll, args.occupancy, "ours_us", round(sum(kt) / len(kt) * 1e3, 1))
        return
    best, serial_ms, ref_times = [], 0.0, []
    for f, fs in enumerate(cfg.features):
        kinds = ["onehot"] if fs.length == "onehot" else ["ws", "obms"]
        times = {k: time_alone(f, k) for k in kinds}
        k = min(times, key=times.get)
        best.append(k)
        ref_times.append(times)
        serial_ms += times[k]
    if args.per_feature:
        for f, fs in enumerate(cfg.features):
            one = FeatEmbed(dev, embed_tables=[tables[f]])
            row = {}
            for kind, u, occ in (("stream", 4, 8), ("pipe", 8, 3), ("warp", 8, 8), ("group", 4, 8)):
                one.set_schedules([Schedule(kind, u)], occupancy=occ)
                o1 = torch.empty((B, fs.dim), dtype=torch.float32, device=dev)
                for _ in range(2):
                    one([dv[f]], [do[f]], out=o1)
                one.kernel_timing(True)
                for _ in range(5):
                    one([dv[f]], [do[f]], out=o1)
                kt = one.kernel_times()
                one.kernel_timing(False)
                row[f"{kind}{u}o{occ}"] = round(sum(kt) / len(kt) * 1e3, 1)
            nnz = int(do[f][-1])
            print(f"f{f:02d} dim {fs.dim:3d} rows {fs.rows:8d} len {fs.length}{fs.length_args} idx {fs.index} nnz {nnz:9d} "
                  f"ref_us { {k: round(v * 1e3, 1) for k, v in ref_times[f].items()} } ours_us {row}", flush=True)
    streams = [torch.cuda.Stream(device=dev) for _ in range(16)]

    def all_features():
        main_s = torch.cuda.current_stream()
        for s in streams:
            s.wait_stream(main_s)
        for f, k in enumerate(best):
            launch(f, k, streams[f % len(streams)])
        for s in streams:
            main_s.wait_stream(s)

    for _ in range(3):
        all_features()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.reps):
        all_features()
    e1.record()
    e1.synchronize()
    overlapped_ms = e0.elapsed_time(e1) / args.reps

    mod = FeatEmbed(dev, embed_tables=tables)
    tuned = os.path.join(ROOT, "recflex_b200", "tuned", f"{args.workload}.json")
    if os.path.exists(tuned):
        with open(tuned) as fh:
            t = json.load(fh)
        mod.set_schedules([Schedule.from_json(s) for s in t["schedules"]], occupancy=t["occupancy"])
    out = torch.empty((B, mod.output_units), dtype=torch.float32, device=dev)
    for _ in range(3):
        mod(dv, do, out=out)
    mod.kernel_timing(True)
    e0.record()
    for _ in range(args.reps):
        mod(dv, do, out=out)
    e1.record()
    e1.synchronize()
    ours_step = e0.elapsed_time(e1) / args.reps
    kt = mod.kernel_times()
    ours_kernel = sum(kt) / len(kt)
    # same answer?
    col, max_err = 0, 0.0
    all_features()
    torch.cuda.synchronize()
    for f, fs in enumerate(cfg.features):
        max_err = max(max_err, float((out[:, col:col + fs.dim] - outs[f]).abs().max()))
        col += fs.dim
    print(json.dumps({
        "workload": cfg.name, "batch": B, "features": len(cfg.features),
        "reference_templates_sum_of_best_alone_ms": serial_ms,
        "reference_templates_16_streams_ms": overlapped_ms,
        "reference_picks": {k: best.count(k) for k in set(best)},
        "ours_fused_kernel_ms": ours_kernel, "ours_step_ms": ours_step,
        "speedup_vs_reference_overlapped": overlapped_ms / ours_step,
        "max_abs_difference": max_err,
    }))


if __name__ == "__main__":
    main()
