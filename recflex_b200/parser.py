"""Readers of the reference's text formats (same names and arguments as RecFlex/parser.py).

* `table_config.txt`: one `rows,dim` line per feature (`parse_table_shapes`, parser.py:64-69);
* `schedule_config.txt`: per feature the comma-separated names of its candidate schedule classes
  (`parse_schedule_types`, parser.py:19-26); `SCHEDULE_KINDS` maps the reference's class names to this
  library's schedule kinds;
* `batch_sizes.txt` + `f{i}.txt`: all batches of a feature back to back, one line per sample
  (`parse_raw_data_batches`, parser.py:28-62), sampled with the same numpy calls as the reference so that the
  same seed selects the same batches.

`parse_knl_total_time` (nsys report parsing, parser.py:71-85) has no counterpart: kernel time comes from
CUDA events (`FeatEmbed.kernel_timing`).
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import numpy as np

# reference schedule class (examples/schedules/*.py) -> schedule kind of this library
SCHEDULE_KINDS = {
    "OneHotSchedule": "group",
    "OneHotMultiBlockSchedule": "group",
    "WarpPerSampleSchedule": "group",
    "OneBlockMultiSampleSchedule": "warp",
    "ReduceByKeySchedule": "flat",
    "MultiBlockPerSampleSchedule": "stream",
}


def parse_schedule_types(config_fname: str, schedule_mapping: Dict[str, object] = None, sep: str = ",") -> List[list]:
    """Per feature, the list of candidate schedules named in the file, mapped through `schedule_mapping`
    (default: `SCHEDULE_KINDS`); unknown names map to None, as `dict.get` does in the reference."""
    mapping = SCHEDULE_KINDS if schedule_mapping is None else schedule_mapping
    with open(config_fname) as f:
        return [list(map(mapping.get, line.strip().split(sep))) for line in f.readlines()]


def parse_raw_data_batches(batch_sizes_fname: str, data_fnames: List[str], sample_batch_nums: int = 128, seed: int = 0,
                           feat_major: bool = True) -> List[List[List[str]]]:
    """Sampled batches as lists of strings: (num_feats, sample_batch_nums, batch_size) when `feat_major`,
    else (sample_batch_nums, num_feats, batch_size)."""
    np.random.seed(seed)
    with open(batch_sizes_fname) as f:
        batch_sizes = [int(line.strip()) for line in f.readlines()]
    line_offsets = np.cumsum([0] + batch_sizes)
    sample_batch_nums = min([sample_batch_nums, len(batch_sizes)])
    sample_batch_ids = np.sort(np.random.choice(len(batch_sizes), sample_batch_nums, replace=False))
    out = [[] for _ in range(len(data_fnames) if feat_major else sample_batch_nums)]
    for feat_id, fname in enumerate(data_fnames):
        with open(fname) as f:
            lines = f.read().splitlines()
        for i, batch_id in enumerate(sample_batch_ids):
            chunk = lines[line_offsets[batch_id]:line_offsets[batch_id + 1]]
            if feat_major:
                out[feat_id].append(chunk)
            else:
                out[i].append(chunk)
    return out


def parse_table_shapes(config_fname: str, sep: str = ",") -> List[Tuple[int, int]]:
    with open(config_fname) as f:
        return [tuple(map(int, line.strip().split(sep))) for line in f.readlines()]
