"""Regenerates tests/golden/einsum_trivia_kat.json from a checkout of the reference project.

test/einsum/einsum_trivia_exec.ml:67-84 contracts two `range_of_shape` tensors
(a: 2|3->4, b: 2|4->5) in four ways and test/einsum/einsum_trivia_exec.expected prints the
results.  This script copies the printed cells of those four tables (c, d, e, f), as the
strings the reference printed, into a small fixture: cells[block][row][column-cell][k], where
a block is one outer-axis row of the table, a row one printed line, a column-cell one boxed
group of numbers on that line.

    python tests/golden/make_einsum_kat.py <reference checkout>      (or set OCANNL_REFERENCE)
"""
import json
import os
import re
import sys

NUM = re.compile(r"-?\d+\.\d+(?:e[+-]\d+)?")


def table(lines, label):
    start = next(i for i, ln in enumerate(lines) if ("*._%s shape" % label) in ln)
    shape = lines[start].split("shape", 1)[1].strip(" │\n")
    blocks, cur = [], []
    for ln in lines[start + 1:]:
        if ln.startswith("│└") or ln.startswith("└"):
            break
        if ln.startswith("│├"):
            if cur:
                blocks.append(cur)
            cur = []
            continue
        if not ln.startswith("││"):
            continue
        cells = ln.split("│")[3:-2]
        nums = [NUM.findall(c) for c in cells]
        if any(nums):
            cur.append(nums)
    if cur:
        blocks.append(cur)
    return {"shape": shape, "cells": blocks}


def main(ref):
    path = os.path.join(ref, "test", "einsum", "einsum_trivia_exec.expected")
    lines = open(path, encoding="utf-8").read().splitlines()
    # the tables of interest follow the marker of the first of the five print statements
    lines = lines[next(i for i, ln in enumerate(lines) if ln.startswith("HERE: test/einsum/einsum_trivia_exec.ml:80:")):]
    out = {"source": "test/einsum/einsum_trivia_exec.expected (tables printed for einsum_trivia_exec.ml:80-84)"}
    for label in ("c", "d", "e", "f"):
        out[label] = table(lines, label)
    here = os.path.dirname(os.path.abspath(__file__))
    with open(os.path.join(here, "einsum_trivia_kat.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
        f.write("\n")


if __name__ == "__main__":
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("OCANNL_REFERENCE")
    if not ref:
        sys.exit("usage: make_einsum_kat.py <reference checkout>")
    main(ref)
