"""Two-stage schedule tuner (the counterpart of RecFlex/tuning/tuner.py, measure.py).

Local stage (reference: `Tuner.tune`, tuner.py:112-152; `measure_single_feat`, measure.py:20-58): for every
feature and every candidate occupancy, ONE launch of the fused kernel runs all of the feature's candidate
schedules side by side: the feature's table is replicated once per candidate (the replicas share the table's
device memory) and every replica gets its own copy of the sampled batch with the indices rotated by a different
amount, so that the candidates fill the GPU and compete for DRAM the way different features do in the real
kernel (replicas that read the very same rows would turn the probe into an L2 benchmark: the B200's 126 MB L2
serves 15 of 16 identical gathers).  The per-replica sum of tile clocks (`eb_forward_timed`) ranks the
candidates.  Every candidate is already compiled into the library: there is no code generation, no
compilation and no process spawning (the reference builds one shared object per feature and occupancy).

Global stage (reference: `Tuner.solve` / `tune_occupancy`, tuner.py:154-205): for each occupancy, the per-feature
winners are installed and the fused kernel is timed on the sampled batches with CUDA events
(`eb_kernel_timing`, replacing `nsys stats gpukernsum`); the fastest occupancy wins.

Refinement (no counterpart in the reference, where every trial costs a compilation): starting from the global
stage's result, whole clusters of look-alike features are switched to each of their best local candidates
inside the real fused kernel, and a switch is kept when the kernel gets faster.  The global stage also times a
small portfolio of uniform assignments, so the result is never worse than the best uniform schedule.

Also here: `mutation_validation` (tuner.py:207-247), `tune_naive` (tuner.py:249-310; candidates timed one
at a time on an otherwise idle GPU), clustering of look-alike features so that one representative is tuned
per cluster (examples/compress.py:28-80), JSON persistence of the result, and `needs_retune` for inputs whose
length statistics moved (distribution shift).
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import _lib
from .rec_modules import FeatEmbed, Schedule

KINDS = ("group", "warp", "flat", "stream", "pipe")
UNROLLS = (1, 2, 4, 6, 8)


@dataclass
class TuneConfig:
    """Search space and effort (reference: `TuneConfig`, tuner.py:38-46, and each schedule's GenParamCandidates)."""

    occupancies: Sequence[int] = (2, 3, 4, 5, 6, 8)
    kinds: Sequence[str] = KINDS
    unrolls: Sequence[int] = UNROLLS
    reps: int = 2                 # launches per (feature, occupancy) in the local stage
    global_reps: int = 3          # passes over the sampled batches per occupancy in the global stage
    min_replicas: int = 16        # candidates are repeated until at least this many replicas fill the GPU
    cluster: bool = True          # tune one representative per cluster of look-alike features
    max_probe_bytes: int = 2 << 30  # cap of the local stage's output buffer
    uniform_portfolio: Sequence[Tuple[str, int]] = (("stream", 2), ("stream", 4), ("stream", 8), ("warp", 4),
                                                    ("pipe", 2), ("pipe", 4), ("pipe", 6), ("pipe", 8))
    hybrid_min_len: Sequence[int] = (32, 128)  # warp-per-bag kernel for features whose mean bag is at least this long
    overlaps: Sequence[int] = (1, 2, 3)  # fused-kernel CTAs per SM tried with the warp-per-bag kernel beside it
    refine_top: int = 3           # local-stage candidates tried per cluster in the refinement pass (0 = off)
    refine_min_gain: float = 0.003  # a switch must make the fused kernel this much faster (relative) to be kept


@dataclass
class InputStats:
    """Per-feature statistics of the sampled batches (what the candidates' ranking depends on)."""

    mean_len: float
    max_len: int
    empty_frac: float

    def bucket(self) -> Tuple[int, int]:
        return (int(round(math.log2(max(self.mean_len, 0.25)))), int(round(math.log2(max(self.max_len, 1)))))


@dataclass
class TuneResult:
    schedules: List[Schedule]
    occupancy: int
    local_times: Dict[int, Dict[int, List[float]]] = field(default_factory=dict)   # feature -> occupancy -> per candidate
    global_ms: Dict[int, float] = field(default_factory=dict)                       # occupancy -> fused-kernel ms
    stats: List[InputStats] = field(default_factory=list)
    overlap: int = 0   # > 0: fused kernel on this many CTAs per SM, warp-per-bag kernel beside it (set_kernel_overlap)

    def to_json(self) -> dict:
        return {
            "occupancy": self.occupancy,
            "overlap": self.overlap,
            "schedules": [s.to_json() for s in self.schedules],
            "global_ms": {str(k): v for k, v in self.global_ms.items()},
            "stats": [[s.mean_len, s.max_len, s.empty_frac] for s in self.stats],
        }

    def save(self, path: str, **extra) -> None:
        d = self.to_json()
        d.update(extra)
        with open(path, "w") as f:
            json.dump(d, f, indent=1)

    @staticmethod
    def load(path: str) -> "TuneResult":
        with open(path) as f:
            d = json.load(f)
        return TuneResult(
            schedules=[Schedule.from_json(s) for s in d["schedules"]],
            occupancy=int(d["occupancy"]),
            global_ms={int(k): float(v) for k, v in d.get("global_ms", {}).items()},
            stats=[InputStats(*s) for s in d.get("stats", [])],
            overlap=int(d.get("overlap", 0)),
        )

    def apply(self, module: FeatEmbed) -> None:
        """Install the schedules, the occupancy and the kernel-overlap setting on `module`."""
        module.set_schedules(self.schedules, occupancy=self.occupancy)
        module.set_kernel_overlap(self.overlap)


def tuned_path(workload: str) -> str:
    """Where the committed tuning result of a benchmark workload ('cfg2', 'cfg3', ...) lives."""
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "tuned", f"{workload}.json")


def input_stats(offsets: Sequence[torch.Tensor]) -> List[InputStats]:
    """Statistics of one batch: offsets[f] has batch + 1 entries (host or device)."""
    out = []
    for o in offsets:
        lens = (o[1:] - o[:-1]).to(torch.float64)
        if lens.numel() == 0:
            out.append(InputStats(0.0, 0, 1.0))
        else:
            out.append(InputStats(float(lens.mean()), int(lens.max()), float((lens == 0).to(torch.float64).mean())))
    return out


def needs_retune(old: Sequence[InputStats], new: Sequence[InputStats]) -> List[int]:
    """Features whose length statistics moved to another bucket since they were tuned."""
    return [f for f, (a, b) in enumerate(zip(old, new)) if a.bucket() != b.bucket()]


class Tuner:
    """Tunes a `FeatEmbed` on sampled batches.  `batches` is a list of (values, offsets) per-feature tensor lists
    on the module's device, offsets with batch + 1 entries (reference: `Tuner.__init__`, tuner.py:49-81, which
    loads `sample_batch_nums` batches from the data files)."""

    def __init__(self, module: FeatEmbed, batches: Sequence[Tuple[Sequence[torch.Tensor], Sequence[torch.Tensor]]],
                 config: Optional[TuneConfig] = None, candidates_from: Optional[Sequence[Sequence[Optional[str]]]] = None):
        """`candidates_from`: per feature, the schedule kinds it may use (what `parser.parse_schedule_types` returns
        for a `schedule_config.txt`; unknown names arrive as None and are ignored).  The reference restricts every
        feature's candidates to the classes its schedule_config line names (tuner.py:70-81)."""
        if not batches:
            raise ValueError("at least one sampled batch is needed")
        if candidates_from is not None and len(candidates_from) != module.num_features:
            raise ValueError(f"candidates_from has {len(candidates_from)} entries for {module.num_features} features")
        self.candidates_from = None if candidates_from is None else [
            tuple(dict.fromkeys(k for k in kinds if k is not None)) for kinds in candidates_from]
        self.module = module
        self.batches = list(batches)
        self.config = config or TuneConfig()
        self.num_feats = module.num_features
        stats = [input_stats(o) for _, o in self.batches]
        self.stats = [
            InputStats(sum(s[f].mean_len for s in stats) / len(stats), max(s[f].max_len for s in stats),
                       sum(s[f].empty_frac for s in stats) / len(stats)) for f in range(self.num_feats)
        ]
        self._probe_out = None
        self._cands: Dict[int, List[Schedule]] = {}   # candidates each feature was measured with

    # -- search space ------------------------------------------------------
    def candidates(self, feat: int) -> List[Schedule]:
        """Candidate schedules of one feature (reference: `gen_feat_sched_param_candidates`, tuner.py:76-81)."""
        st = self.stats[feat]
        cands = []
        kinds = self.config.kinds
        if self.candidates_from is not None:
            kinds = self.candidates_from[feat]
            if not kinds:
                raise ValueError(f"feature {feat}: the schedule configuration names no schedule this library knows")
        for kind in kinds:
            for u in self.config.unrolls:
                if kind == "group" and st.mean_len > 64:
                    continue  # a slot walking hundreds of rows alone leaves the other slots idle
                if kind == "group" and u > 1 and st.max_len <= 1:
                    continue  # one-hot: a bag never has a second row to keep in flight
                if kind == "pipe" and u == 1:
                    continue  # the ring's shallowest variant is unroll 2
                if u == 6 and kind != "pipe":
                    continue  # six rows per macro-step exist for the ring only (48 KB of it: 4 CTAs per SM)
                if kind == "warp" and u not in (2, 4):
                    continue  # the warp-per-bag kernel keeps two or four rows per lane in flight
                cands.append(Schedule(kind, u))
        return cands

    def clusters(self) -> Dict[tuple, List[int]]:
        """Features that look alike to the kernel (reference idea: examples/compress.py:28-80)."""
        groups: Dict[tuple, List[int]] = {}
        for f, t in enumerate(self.module.embed_tables):
            key = (f,)
            if self.config.cluster:
                key = (int(t.shape[1]), str(t.dtype), int(round(math.log2(max(int(t.shape[0]), 1)) / 2)),
                       self.stats[f].bucket(), self.candidates_from[f] if self.candidates_from is not None else None)
            groups.setdefault(key, []).append(f)
        return groups

    # -- local stage -------------------------------------------------------
    def _probe(self, feat: int, cands: Sequence[Schedule], occupancy: int, replicas: int):
        table = self.module.embed_tables[feat]
        probe = FeatEmbed(self.module.device, embed_tables=[table] * replicas)
        probe.set_schedules([cands[i % len(cands)] for i in range(replicas)], occupancy=occupancy)
        return probe

    def measure_feature(self, feat: int, occupancy: int, cands: Optional[Sequence[Schedule]] = None) -> List[float]:
        """Summed tile time (ms) of every candidate of `feat` at `occupancy`, all candidates in one launch."""
        cands = list(cands or self.candidates(feat))
        table = self.module.embed_tables[feat]
        batch = self.batches[0][1][feat].numel() - 1
        row_out = int(table.shape[1]) * 4 * max(batch, 1)
        replicas = max(self.config.min_replicas, len(cands))
        replicas = (replicas + len(cands) - 1) // len(cands) * len(cands)  # padded by repetition (tuner.py:83-91)
        while replicas > len(cands) and replicas * row_out > self.config.max_probe_bytes:
            replicas -= len(cands)
        probe = self._probe(feat, cands, occupancy, replicas)
        need = batch * probe.output_units
        if self._probe_out is None or self._probe_out.numel() < need:
            self._probe_out = torch.empty(need, dtype=torch.float32, device=self.module.device)
        out = self._probe_out[:need].view(batch, probe.output_units)
        totals = [0.0] * len(cands)
        rows = int(table.shape[0])
        for values, offsets in self.batches:
            v, o = values[feat], offsets[feat]
            # replica i reads rows rotated by i * rows / replicas: same popularity profile, different DRAM lines
            vs = [v if i == 0 else torch.remainder(v + (i * rows) // replicas, rows).to(v.dtype)
                  for i in range(replicas)]
            for _ in range(self.config.reps):
                _, times = probe(vs, [o] * replicas, timing=True, out=out)
                for i in range(replicas):
                    totals[i % len(cands)] += float(times[i])
        return totals

    def tune_local(self) -> Dict[int, Dict[int, List[float]]]:
        """feature -> occupancy -> per-candidate time (reference: `Tuner.tune`)."""
        results: Dict[int, Dict[int, List[float]]] = {}
        for members in self.clusters().values():
            rep = members[0]
            cands = self.candidates(rep)
            per_occ = {occ: self.measure_feature(rep, occ, cands) for occ in self.config.occupancies}
            for f in members:
                results[f] = per_occ
                self._cands[f] = cands
        return results

    # -- global stage ------------------------------------------------------
    def fused_ms(self, schedules: Sequence[Schedule], occupancy: int, reps: Optional[int] = None) -> float:
        """Mean fused-kernel milliseconds over the sampled batches with `schedules` installed."""
        mod = self.module
        mod.set_schedules(schedules, occupancy=occupancy)
        for values, offsets in self.batches:  # warm-up
            mod(values, offsets)
        mod.kernel_timing(True)
        for _ in range(reps or self.config.global_reps):
            for values, offsets in self.batches:
                mod(values, offsets)
        times = mod.kernel_times()
        mod.kernel_timing(False)
        return sum(times) / max(len(times), 1)

    def solve(self, local: Dict[int, Dict[int, List[float]]]) -> TuneResult:
        """Per occupancy pick every feature's fastest candidate, then pick the occupancy (reference: `Tuner.solve`)."""
        feat_cands = {f: self._cands.get(f) or self.candidates(f) for f in range(self.num_feats)}
        global_ms, winners = {}, {}
        for occ in self.config.occupancies:
            scheds = []
            for f in range(self.num_feats):
                t = local[f][occ]
                scheds.append(feat_cands[f][min(range(len(t)), key=t.__getitem__)])
            winners[occ] = scheds
            global_ms[occ] = self.fused_ms(scheds, occ)
            best_uni, best_uni_ms = None, float("inf")
            for kind, unroll in self.config.uniform_portfolio:  # never end up worse than a uniform assignment
                uni = [Schedule(kind, unroll) for _ in range(self.num_feats)]
                ms = self.fused_ms(uni, occ)
                if ms < global_ms[occ]:
                    global_ms[occ], winners[occ] = ms, uni
                if kind != "warp" and ms < best_uni_ms:
                    best_uni, best_uni_ms = uni, ms
            for mix in self.hybrids(best_uni):
                ms = self.fused_ms(mix, occ)
                if ms < global_ms[occ]:
                    global_ms[occ], winners[occ] = ms, mix
        best = min(global_ms, key=global_ms.get)
        self.module.set_schedules(winners[best], occupancy=best)
        return TuneResult(winners[best], best, local, global_ms, self.stats)

    def hybrids(self, base: Optional[Sequence[Schedule]]) -> List[List[Schedule]]:
        """Assignments that send long bags to the warp-per-bag kernel and leave everything else as in `base`.  The
        local stage ranks a feature's candidates inside ONE kernel and cannot see this split."""
        out = []
        for min_len in self.config.hybrid_min_len:
            long_bags = [f for f in range(self.num_feats) if self.stats[f].mean_len >= min_len]
            if base is None or not long_bags or len(long_bags) == self.num_feats:
                continue
            mix = list(base)
            for f in long_bags:
                mix[f] = Schedule("warp", 4)
            out.append(mix)
        return out

    def refine(self, result: TuneResult) -> TuneResult:
        """Greedy pass in the real fused kernel: for each cluster (heaviest first), try its best local candidates
        for the whole cluster and keep a switch that makes the kernel faster."""
        if self.config.refine_top <= 0 or not result.local_times:
            return result
        occ = result.occupancy
        scheds = list(result.schedules)
        best_ms = self.fused_ms(scheds, occ)
        weight = lambda members: -sum(self.stats[f].mean_len * int(self.module.embed_tables[f].shape[1]) *
                                      self.module.embed_tables[f].element_size() for f in members)
        for members in sorted(self.clusters().values(), key=weight):
            rep = members[0]
            cands = self._cands.get(rep) or self.candidates(rep)
            t = result.local_times[rep][occ]
            order = sorted(range(len(cands)), key=t.__getitem__)[: self.config.refine_top]
            tried = {scheds[rep].kind * 16 + scheds[rep].unroll}
            for pick in [cands[i] for i in order] + [Schedule(k, u) for k, u in self.config.uniform_portfolio]:
                key = pick.kind * 16 + pick.unroll
                if key in tried:
                    continue
                tried.add(key)
                trial = list(scheds)
                for f in members:
                    trial[f] = pick
                ms = self.fused_ms(trial, occ, reps=2)
                if ms < best_ms * (1.0 - self.config.refine_min_gain):
                    ms2 = self.fused_ms(trial, occ, reps=2)  # confirm: a single timing can be a fluke
                    if ms2 < best_ms * (1.0 - self.config.refine_min_gain):
                        scheds, best_ms = trial, min(ms, ms2)
        self.module.set_schedules(scheds, occupancy=occ)
        gm = dict(result.global_ms)
        gm[occ] = best_ms
        return TuneResult(scheds, occ, result.local_times, gm, result.stats)

    def tune_overlap(self, result: TuneResult) -> TuneResult:
        """Last step: when the assignment uses both kernels (some features on the warp-per-bag schedule, some not),
        try running them side by side, the fused kernel on a reduced grid, and keep the fastest arrangement."""
        mod = self.module
        n_warp = sum(1 for s in result.schedules if s.kind == _lib.EB_SCHED_WARP)
        mod.set_kernel_overlap(0)
        if n_warp == 0 or n_warp == self.num_feats or not self.config.overlaps:
            return result
        best_n, best_ms = 0, self.fused_ms(result.schedules, result.occupancy)
        for n in self.config.overlaps:
            if n > result.occupancy:
                continue
            mod.set_kernel_overlap(n)
            ms = self.fused_ms(result.schedules, result.occupancy)
            if ms < best_ms * (1.0 - self.config.refine_min_gain):
                best_n, best_ms = n, ms
        mod.set_kernel_overlap(best_n)
        gm = dict(result.global_ms)
        gm[result.occupancy] = best_ms
        return TuneResult(result.schedules, result.occupancy, result.local_times, gm, result.stats, best_n)

    def tune(self) -> TuneResult:
        self.module.set_kernel_overlap(0)
        return self.tune_overlap(self.refine(self.solve(self.tune_local())))

    # -- ablations ---------------------------------------------------------
    def mutation_validation(self, result: TuneResult, feat: int) -> Tuple[List[float], int]:
        """Swap `feat`'s schedule through all of its candidates inside the tuned kernel; returns the fused-kernel
        time of each mutation and the index of the tuner's pick (reference: tuner.py:207-247)."""
        cands = self.candidates(feat)
        times = []
        for c in cands:
            scheds = list(result.schedules)
            scheds[feat] = c
            times.append(self.fused_ms(scheds, result.occupancy))
        pick = next((i for i, c in enumerate(cands) if c == result.schedules[feat]), -1)
        self.module.set_schedules(result.schedules, occupancy=result.occupancy)
        return times, pick

    def tune_naive(self, occupancy: int = 4) -> TuneResult:
        """Pick every feature's candidate by timing it alone on an idle GPU (reference: `tune_naive`,
        tuner.py:249-310): no interference between features is modelled."""
        scheds = []
        for f in range(self.num_feats):
            cands = self.candidates(f)
            table = self.module.embed_tables[f]
            probe = FeatEmbed(self.module.device, embed_tables=[table])
            best, best_ms = cands[0], float("inf")
            for c in cands:
                probe.set_schedules([c], occupancy=occupancy)
                probe.kernel_timing(True)
                for values, offsets in self.batches:
                    probe([values[f]], [offsets[f]])
                t = probe.kernel_times()
                probe.kernel_timing(False)
                ms = sum(t) / max(len(t), 1)
                if ms < best_ms:
                    best, best_ms = c, ms
            scheds.append(best)
        ms = self.fused_ms(scheds, occupancy)
        return TuneResult(scheds, occupancy, {}, {occupancy: ms}, self.stats)

    def tune_fixed_thread_binding(self, result: TuneResult, choice: str = "max") -> Tuple[List[int], float, float]:
        """Ablation (reference: `tune_fixed_thread_binding`, tuner.py:312-357): replace the per-batch binding by a
        fixed one.  The tile counts the device chose for every sampled batch under `result`'s schedules are reduced
        per feature to their maximum or mean (`choice`), turned back into a fixed bags-per-tile, installed, and the
        kernel is timed.  Returns (fixed bags per tile, kernel ms with the fixed binding, kernel ms with the
        run-time binding); `result`'s schedules are back in place afterwards."""
        if choice not in ("max", "mean"):
            raise ValueError("choice must be 'max' or 'mean'")
        mod = self.module
        result.apply(mod)
        tiles = []
        for values, offsets in self.batches:
            mod(values, offsets)
            batch = offsets[0].numel() - 1
            tiles.append([-(-batch // n) for n in mod.last_binding()])
        fixed = []
        for f in range(self.num_feats):
            per_batch = [t[f] for t in tiles]
            want = max(per_batch) if choice == "max" else max(1, sum(per_batch) // len(per_batch))
            batch = self.batches[0][1][f].numel() - 1
            n = max(1, min(1024, batch // max(want, 1)))
            fixed.append(1 << (n.bit_length() - 1))  # bags per tile are powers of two
        dynamic_ms = self.fused_ms(result.schedules, result.occupancy)
        pinned = [Schedule(s.kind, s.unroll, fixed[f]) for f, s in enumerate(result.schedules)]
        fixed_ms = self.fused_ms(pinned, result.occupancy)
        result.apply(mod)
        return fixed, fixed_ms, dynamic_ms

    def retune(self, result: TuneResult, new_batches) -> TuneResult:
        """Re-run the local stage only for features whose statistics moved bucket on `new_batches`, keep the
        occupancy sweep (distribution shift)."""
        self.module.set_kernel_overlap(0)
        fresh = Tuner(self.module, new_batches, self.config, self.candidates_from)
        moved = set(needs_retune(result.stats, fresh.stats)) if result.stats else set(range(self.num_feats))
        if not moved:
            fresh.module.set_schedules(result.schedules, occupancy=result.occupancy)
            fresh.module.set_kernel_overlap(result.overlap)
            return TuneResult(result.schedules, result.occupancy, {}, {}, fresh.stats, result.overlap)
        local: Dict[int, Dict[int, List[float]]] = {}
        for members in fresh.clusters().values():
            todo = [f for f in members if f in moved]
            if not todo:
                continue
            cands = fresh.candidates(todo[0])
            per_occ = {occ: fresh.measure_feature(todo[0], occ, cands) for occ in self.config.occupancies}
            for f in todo:
                local[f] = per_occ
                fresh._cands[f] = cands
        global_ms, winners = {}, {}
        for occ in self.config.occupancies:
            scheds = list(result.schedules)
            for f in moved:
                t = local[f][occ]
                scheds[f] = fresh._cands[f][min(range(len(t)), key=t.__getitem__)]
            winners[occ] = scheds
            global_ms[occ] = fresh.fused_ms(scheds, occ)
            for mix in fresh.hybrids(scheds):
                ms = fresh.fused_ms(mix, occ)
                if ms < global_ms[occ]:
                    global_ms[occ], winners[occ] = ms, mix
        best = min(global_ms, key=global_ms.get)
        self.module.set_schedules(winners[best], occupancy=best)
        return fresh.tune_overlap(TuneResult(winners[best], best, local, global_ms, fresh.stats))


def main(argv=None) -> None:
    """Command line: tune one of the synthetic benchmark configurations and write the result as JSON
    (reference: examples/tune.py:96-122).

        python -m recflex_b200.tuning --workload cfg3 --out recflex_b200/tuned/cfg3.json
    """
    import argparse
    import time

    from . import synth

    p = argparse.ArgumentParser(description=main.__doc__)
    p.add_argument("--workload", default="cfg3", choices=["cfg1", "cfg2", "cfg3", "cfg4", "cfg5"])
    p.add_argument("--row-scale", type=float, default=1.0)
    p.add_argument("--batch", type=int, default=0)
    p.add_argument("--sample-batches", type=int, default=2)
    p.add_argument("--occupancies", type=str, default="3,4,5,6,8")
    p.add_argument("--naive", action="store_true", help="ablation: time candidates alone (no interference)")
    p.add_argument("--mutation-feat-id", type=int, default=-1)
    p.add_argument("--no-cluster", action="store_true")
    p.add_argument("--schedule-config", type=str, default="",
                   help="a schedule_config.txt of the reference: restricts every feature's candidates to the classes "
                        "its line names (mapped to this library's kinds by parser.SCHEDULE_KINDS)")
    p.add_argument("--fixed-thread-binding", choices=["", "max", "mean"], default="",
                   help="ablation: also time the tuned kernel with a fixed bags-per-tile per feature")
    p.add_argument("--out", type=str, required=True)
    args = p.parse_args(argv)

    dev = torch.device("cuda", torch.cuda.current_device())
    cfg = synth.make_config(int(args.workload[3:]), row_scale=args.row_scale, batch=args.batch or None)
    tables = synth.make_tables_device(cfg, dev)
    mod = FeatEmbed(dev, embed_tables=tables)
    batches = []
    for i in range(args.sample_batches):
        v, o = synth.gen_batch(cfg, seed=7000 + i)
        batches.append(([torch.from_numpy(x).to(dev) for x in v], [torch.from_numpy(x).to(dev) for x in o]))
    tc = TuneConfig(occupancies=tuple(int(x) for x in args.occupancies.split(",")), cluster=not args.no_cluster)
    allowed = None
    if args.schedule_config:
        from .parser import parse_schedule_types

        allowed = parse_schedule_types(args.schedule_config)
    tuner = Tuner(mod, batches, tc, candidates_from=allowed)
    t0 = time.time()
    base_ms = tuner.fused_ms([Schedule("auto") for _ in range(mod.num_features)], 4)
    res = tuner.tune_naive() if args.naive else tuner.tune()
    extra = {"workload": cfg.name, "default_ms": base_ms, "tuned_ms": res.global_ms.get(res.occupancy),
             "tuning_seconds": time.time() - t0, "clusters": len(tuner.clusters()),
             "device": torch.cuda.get_device_name(dev)}
    if args.mutation_feat_id >= 0:
        times, pick = tuner.mutation_validation(res, args.mutation_feat_id)
        extra["mutation"] = {"feature": args.mutation_feat_id, "times_ms": times, "pick": pick}
    if args.fixed_thread_binding:
        fixed, fixed_ms, dyn_ms = tuner.tune_fixed_thread_binding(res, args.fixed_thread_binding)
        extra["fixed_thread_binding"] = {"choice": args.fixed_thread_binding, "bags_per_tile": fixed,
                                         "fixed_ms": fixed_ms, "runtime_binding_ms": dyn_ms}
    res.save(args.out, **extra)
    print(json.dumps({k: v for k, v in extra.items() if k != "mutation"}))
    print("occupancy", res.occupancy, "global_ms", res.global_ms)


if __name__ == "__main__":
    main()
