"""Regenerates tests/golden/cc_golden_digests.json from a checkout of the reference project.

For each golden generated-C file of the reference, takes the text of the routine
(from its ` void <name>(` line to the end of the file), removes all whitespace and
records the SHA-256 and length.  The parity test recomputes the same digest from
the oracle emitter's output, so the golden text itself never enters this repository.

One more entry comes from the C listing in docs/slides-basics_backprop_training_codegen.md
(the materialised-accumulate contraction printed as an `fmaf` nest, `fmaxf(0.0, ...)` and the
SGD assignment): the statements between `/* Main logic. */` and the end of the function, with
the listing's `...` elision lines dropped.

    python tests/golden/make_cc_golden_digests.py <reference checkout>
    (or set OCANNL_REFERENCE to the checkout)
"""
import hashlib
import json
import os
import re
import sys


def routine_text(c_text: str) -> str:
    m = re.search(r"^ ?void \w+\(", c_text, re.M)
    return re.sub(r"\s+", "", c_text[m.start():])


def main_logic_text(c_text: str) -> str:
    """Whitespace-free text from `/* Main logic. */` to the end of the function."""
    at = c_text.index("/* Main logic. */")
    return re.sub(r"\s+", "", c_text[at:])


def slides_listing(md_text: str) -> str:
    at = md_text.index("### C code: `scalar_loss_gradient_then_gd_update.c`")
    block = md_text[md_text.index("```", at) + 3:]
    block = block[:block.index("```")]
    lines = [ln for ln in block.splitlines() if ln.strip() != "..."]
    return main_logic_text("\n".join(lines))


def main(ref):
    out = {}
    for name in ("top_down_prec", "zero_out_local_decl", "test_where_precision"):
        path = os.path.join(ref, "test", "operations", name + ".c.expected")
        t = routine_text(open(path).read())
        out[name] = {"source": "test/operations/%s.c.expected" % name,
                     "sha256": hashlib.sha256(t.encode()).hexdigest(), "chars": len(t)}
    t = slides_listing(open(os.path.join(ref, "docs", "slides-basics_backprop_training_codegen.md")).read())
    out["slides_gd_update"] = {"source": "docs/slides-basics_backprop_training_codegen.md (C listing, main logic)",
                               "sha256": hashlib.sha256(t.encode()).hexdigest(), "chars": len(t)}
    here = os.path.dirname(os.path.abspath(__file__))
    with open(os.path.join(here, "cc_golden_digests.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
        f.write("\n")


if __name__ == "__main__":
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("OCANNL_REFERENCE")
    if not ref:
        sys.exit("usage: make_cc_golden_digests.py <reference checkout>")
    main(ref)
