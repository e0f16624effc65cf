"""Extract the reference's committed golden hashes for the matrix-product path.

Run once where the reference checkout is mounted:

    python tests/golden/make_golden.py /path/to/reference

It copies HASHES ONLY (no source, no data) into small JSON fixtures beside
this script:

  gemm_identical_card.json   the 60 records of the reference's GEMM identity
                             card (bench/results/e1/2026-08-28_131651-runpod-nvidia/
                             lanes/gemm.identical.card): tag, dtype, count, FNV-1a64.
  verify_table_cells.json    the reference cells of the verify table
                             (python/mojolearn/verify_reference/table.json) for the
                             lanes on this path, every fixture, plus the table's own
                             fixture hashes.

The tests read these files only; nothing at test time touches the reference.
"""
import json
import os
import sys

LANES = ["gemm-pinned", "gemm-transposed", "gemm-bf16", "gemm-int8", "gemm-int15", "lowbit-conversions",
         "transformer", "transformer-bf16w", "transformer-int8w", "transformer-window", "transformer-decode-session", "embedding", "hf-causal-lm"]


def main(ref):
    here = os.path.dirname(os.path.abspath(__file__))
    card = []
    path = os.path.join(ref, "bench/results/e1/2026-08-28_131651-runpod-nvidia/lanes/gemm.identical.card")
    with open(path) as fh:
        for line in fh:
            if line.startswith("#") or not line.strip():
                continue
            seq, tag, dtype, count, digest = line.rstrip("\n").split("\t")
            card.append({"seq": int(seq), "tag": tag, "dtype": dtype, "count": int(count), "fnv1a64": digest})
    with open(os.path.join(here, "gemm_identical_card.json"), "w") as fh:
        json.dump({"source": "bench/results/e1/2026-08-28_131651-runpod-nvidia/lanes/gemm.identical.card",
                   "records": card}, fh, indent=1)
    with open(os.path.join(ref, "python/mojolearn/verify_reference/table.json")) as fh:
        table = json.load(fh)
    cells = {}
    for key, cell in table["cells"].items():
        lane, fx = key.split("/")
        if lane not in LANES:
            continue
        kept = {col: v["ref"] for col, v in cell.items() if not str(v.get("ref")).startswith("n/a")}
        cells[key] = kept
    out = {"source": "python/mojolearn/verify_reference/table.json", "format": table["format"],
           "fixtures": table["fixtures"], "heldout": table["heldout"], "cells": cells}
    with open(os.path.join(here, "verify_table_cells.json"), "w") as fh:
        json.dump(out, fh, indent=1, sort_keys=True)
    print("card records:", len(card), "table cells:", len(cells))


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py /path/to/reference")
    main(sys.argv[1])
