"""Generates the golden fixtures of tests/golden/ from the RecFlex reference itself.

Run in a container that has the reference checkout (path as argument or in $RECFLEX_REF) and
after `bash oracle/build_ref.sh`:

    python tests/golden/make_golden.py [/path/to/RecFlex]

* pool_golden.npz — small multi-feature batches (text lines, tables) and the
  expected [batch, sum(dim)] output computed with the formula of the reference's
  own checker (examples/test.py:68-86: per feature and sample
  `F.embedding(LongTensor(indices), table).sum(0)`, empty line -> zeros,
  features side by side).  The reference's `check_results` function, imported
  from the checkout, is then run on that output as a cross-check.
* parse_golden.json — text lines and the (indices, segment_offsets, num_tiles,
  num_blocks) that the reference's compiled host parsers return for them
  (ws::StringSplitToInt, examples/csrc/warp_per_sample_preprocess.cu:6-38;
  onehot::OneHotMultiBlock, examples/csrc/onehot_preprocess.cu:17-27), called
  through oracle/_ref/libref_host.so; plus a tiny model directory in the reference's text formats and what the
  reference's readers (RecFlex/parser.py: parse_table_shapes, parse_raw_data_batches) return for it.

The fixtures are committed; the tests never read the reference checkout.
"""
import ctypes as C
import json
import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("RECFLEX_REF")
if not REF or not os.path.isdir(REF):
    raise SystemExit("usage: make_golden.py <path to the RecFlex checkout>  (or set RECFLEX_REF)")
sys.dont_write_bytecode = True
sys.path.insert(0, REF)
sys.path.insert(0, os.path.join(REF, "examples"))


def reference_formula(tables, raw_data):
    """examples/test.py:68-86, producing the expected tensor instead of asserting."""
    batch = len(raw_data[0])
    cols = []
    for raw, table in zip(raw_data, tables):
        res = torch.zeros((batch, table.shape[1]), dtype=torch.float32)
        for sid, row in enumerate(raw):
            indices = [] if row == "" else list(map(int, row.strip().split(",")))
            res[sid] = F.embedding(torch.LongTensor(indices), table).sum(0)
        cols.append(res)
    return torch.cat(cols, dim=1)


def make_case(rng, dims, rows, batch, max_len, empty_frac, dtype):
    tables, raw = [], []
    for d, r in zip(dims, rows):
        t = torch.from_numpy((rng.standard_normal((r, d)) * 0.05).astype(np.float32))
        if dtype == "f16":
            t = t.half()
        tables.append(t)
        lines = []
        for _ in range(batch):
            if rng.random() < empty_frac:
                lines.append("")
            else:
                n = int(rng.integers(1, max_len + 1))
                lines.append(",".join(str(int(x)) for x in rng.integers(0, r, n)))
        raw.append(lines)
    return tables, raw


def main():
    import test as ref_test  # the reference's examples/test.py

    rng = np.random.default_rng(20241125)
    out = {}
    cases = [
        ("mixed_f32", [4, 8, 16, 32, 64, 128], [37, 64, 100, 211, 150, 90], 24, 9, 0.15, "f32"),
        ("long_f32", [16, 16, 128], [300, 17, 50], 7, 400, 0.2, "f32"),
        ("onehot_f32", [16, 64], [128, 33], 40, 1, 0.0, "f32"),
        ("mixed_f16", [8, 16, 32, 64, 128, 256], [45, 80, 60, 120, 30, 25], 19, 12, 0.1, "f16"),
    ]
    for name, dims, rows, batch, max_len, empty_frac, dtype in cases:
        tables, raw = make_case(rng, dims, rows, batch, max_len, empty_frac, dtype)
        tables_f32 = [t.float() for t in tables]  # fp16 tables: fp32 accumulation over the up-cast values
        expect = reference_formula(tables_f32, raw)
        ref_test.check_results(expect.flatten(), tables_f32, raw)  # the reference's own assertion
        out[f"{name}.expect"] = expect.numpy()
        out[f"{name}.raw"] = np.array(["\n".join(lines) for lines in raw])
        out[f"{name}.batch"] = np.array(batch)
        for i, t in enumerate(tables):
            out[f"{name}.table{i}"] = t.numpy()
    np.savez_compressed(os.path.join(HERE, "pool_golden.npz"), **out)

    lib = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libref_host.so"))
    lib.ref_ws_parse.restype = C.c_int64
    lib.ref_onehot_parse.restype = C.c_int64
    texts = [
        ["3,17,5", "", "42", "0,0,0", "9,8,7,6,5,4,3,2,1,0"],
        ["3,,5", " 7", "8 ", "1;2|3", "12a34", ""],
        ["", "", ""],
        ["2147483647", "000123", "5,"],
        [",".join(str(i) for i in range(300))],
    ]
    parsed = []
    for lines in texts:
        text = "\n".join(lines).encode()
        cap = len(text) + 2
        vals = np.zeros(cap, dtype=np.int32)
        offs = np.zeros(len(lines) + 1, dtype=np.int32)
        tiles, blocks = C.c_int32(), C.c_int32()
        n = lib.ref_ws_parse(text, C.c_int64(len(text)), C.c_int64(len(lines)), 8, vals.ctypes.data_as(C.c_void_p),
                             C.c_int64(cap), offs.ctypes.data_as(C.c_void_p), C.byref(tiles), C.byref(blocks))
        assert n >= 0
        parsed.append({"lines": lines, "tile_size": 8, "indices": vals[:n].tolist(), "segment_offsets": offs.tolist(),
                       "num_tiles": tiles.value, "num_blocks": blocks.value})
    onehot_lines = ["5", "0", "77", "123456", "9"]
    text = "\n".join(onehot_lines).encode()
    vals = np.zeros(len(onehot_lines), dtype=np.int32)
    tiles, blocks = C.c_int32(), C.c_int32()
    n = lib.ref_onehot_parse(text, C.c_int64(len(text)), C.c_int64(len(onehot_lines)), 592, 256,
                             vals.ctypes.data_as(C.c_void_p), C.byref(tiles), C.byref(blocks))
    onehot = {"lines": onehot_lines, "indices": vals[:n].tolist(), "num_tiles": tiles.value, "num_blocks": blocks.value}
    # the reference's text-format readers (RecFlex/parser.py) on a tiny generated model directory
    import tempfile

    from RecFlex.parser import parse_raw_data_batches, parse_table_shapes

    frng = np.random.default_rng(99)
    batch_sizes = [int(x) for x in frng.integers(1, 6, 9)]
    files = {"batch_sizes.txt": "\n".join(map(str, batch_sizes)) + "\n", "table_config.txt": "100,16\n57,8\n300,32\n"}
    for i, rows in enumerate([100, 57, 300]):
        lines = []
        for _ in range(sum(batch_sizes)):
            n = int(frng.integers(0, 4))
            lines.append(",".join(str(int(x)) for x in frng.integers(0, rows, n)))
        files[f"f{i}.txt"] = "\n".join(lines) + "\n"
    with tempfile.TemporaryDirectory() as d:
        for name, text in files.items():
            with open(os.path.join(d, name), "w") as f:
                f.write(text)
        fnames = [os.path.join(d, f"f{i}.txt") for i in range(3)]
        formats = {
            "files": files,
            "table_shapes": [list(t) for t in parse_table_shapes(os.path.join(d, "table_config.txt"))],
            "feat_major": parse_raw_data_batches(os.path.join(d, "batch_sizes.txt"), fnames, 4, seed=3),
            "batch_major": parse_raw_data_batches(os.path.join(d, "batch_sizes.txt"), fnames, 4, seed=3,
                                                  feat_major=False),
        }
    with open(os.path.join(HERE, "parse_golden.json"), "w") as f:
        json.dump({"ws": parsed, "onehot": onehot, "formats": formats}, f, indent=1)
    print("wrote", os.listdir(HERE))


if __name__ == "__main__":
    main()
