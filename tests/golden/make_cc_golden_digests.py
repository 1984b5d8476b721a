"""Regenerates tests/golden/cc_golden_digests.json from the reference checkout.

For each golden generated-C file of the reference, takes the text of the routine
(from its ` void <name>(` line to the end of the file), removes all whitespace and
records the SHA-256 and length.  The parity test recomputes the same digest from
the oracle emitter's output, so the golden text itself never enters this repository.

    python tests/golden/make_cc_golden_digests.py <reference checkout>
"""
import hashlib
import json
import os
import re
import sys


def routine_text(c_text: str) -> str:
    m = re.search(r"^ ?void \w+\(", c_text, re.M)
    return re.sub(r"\s+", "", c_text[m.start():])


def main(ref):
    out = {}
    for name in ("top_down_prec", "zero_out_local_decl", "test_where_precision"):
        path = os.path.join(ref, "test", "operations", name + ".c.expected")
        t = routine_text(open(path).read())
        out[name] = {"source": "test/operations/%s.c.expected" % name,
                     "sha256": hashlib.sha256(t.encode()).hexdigest(), "chars": len(t)}
    here = os.path.dirname(os.path.abspath(__file__))
    with open(os.path.join(here, "cc_golden_digests.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
        f.write("\n")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
