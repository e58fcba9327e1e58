"""Generate tests/golden/gfg_case/ by running the UNMODIFIED reference.

    make -C oracle            # builds oracle/_ref/libtiga_runtime.so from the reference's sources
    python tests/golden/make_golden_gfg.py  [--reference /path/to/TIGA-lang]

Writes two persistent graphs with the reference's own ``tg.save`` -- a ragged int32 CSR without
fields (format v1) and the same relation as int64 with one field per role (format v2) -- and a
small JSON with what the reference's ``tg.load(...)`` reports for them (extents, ``paged_rows`` /
``paged_page`` of a row range).  The directories are committed as fixtures: the reader of this
package must load them, and its writer must reproduce them byte for byte.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", default=os.environ.get("TIGA_REFERENCE"))
    args = parser.parse_args()
    reference = args.reference or os.path.join(os.path.dirname(ROOT), "reference")
    if not os.path.isdir(reference):
        raise SystemExit("pass --reference /path/to/TIGA-lang (or set TIGA_REFERENCE)")
    runtime = os.path.join(ROOT, "oracle", "_ref", "libtiga_runtime.so")
    if not os.path.exists(runtime):
        raise SystemExit("build oracle/_ref first: make -C oracle")
    os.environ["TIGA_RUNTIME_LIBRARY"] = runtime
    sys.dont_write_bytecode = True
    sys.path.insert(0, os.path.join(reference, "python"))
    import tiga as tg

    assert os.path.realpath(tg.__file__).startswith(os.path.realpath(reference))
    out = os.path.join(HERE, "gfg_case")
    shutil.rmtree(out, ignore_errors=True)
    os.makedirs(out)
    row_ptr = [0, 2, 2, 5, 6, 6, 9]                       # two empty rows
    col_idx = [0, 4, 1, 2, 3, 3, 0, 2, 4]
    num_src = 5
    record = {}
    plain = tg.Graph.from_csr(tg.tensor(row_ptr, dtype=tg.int32), tg.tensor(col_idx, dtype=tg.int32),
                              num_src=num_src, validate="full")
    tg.save(plain, os.path.join(out, "plain_i32.gfg"))
    fields = {
        "src": {"x": tg.tensor([[0.5 * i + j for j in range(3)] for i in range(num_src)], dtype=tg.float32)},
        "dst": {"bias": tg.tensor([0.25 * i for i in range(6)], dtype=tg.float32)},
        "edge": {"weight": tg.tensor([1.0 + 0.125 * e for e in range(9)], dtype=tg.float32)},
    }
    wide = tg.Graph.from_csr(tg.tensor(row_ptr, dtype=tg.int64), tg.tensor(col_idx, dtype=tg.int64),
                             num_src=num_src, validate="full")
    tg.save(wide, os.path.join(out, "fields_i64.gfg"), fields=fields)
    for name in ("plain_i32.gfg", "fields_i64.gfg"):
        loaded = tg.load(os.path.join(out, name))
        record[name] = {
            "realization": loaded.schema.realization, "origin": loaded.schema.origin,
            "num_src": loaded.schema.num_src, "num_dst": loaded.schema.num_dst, "num_edges": loaded.num_edges,
            "paged_rows_2_5": [list(part) for part in loaded.paged_rows(2, 5)],
            "paged_page_3_6": [list(part) if isinstance(part, tuple) else part for part in loaded.paged_page(3, 6)],
        }
    with open(os.path.join(out, "expected.json"), "w") as handle:
        json.dump(record, handle, indent=1, sort_keys=True)
    print("wrote", out, sorted(os.listdir(out)))


if __name__ == "__main__":
    main()
