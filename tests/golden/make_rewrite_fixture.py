"""Extracts the INT8 entries of the reference's rename table into tests/golden/rewrite_table.json.

The table lives in itex/core/graph/native_layout/native_layout.cc: entries {"FromOp", "ToOp", CopyAttrsFn, RewriteRuleFn}.
The INT8 entries are in GetCPUEigenNativeFormatInfo (lines 113-199); the reference's GPU build needs no rename for them
because it registers its kernels under the stock names as well.  The fixture keeps every entry of that table whose source
op is a quantized op (name contains "quantize" in either case), with the names of its attr copier and its rule.

    python tests/golden/make_rewrite_fixture.py /path/to/reference
"""
import json
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: %s /path/to/reference-checkout" % os.path.basename(sys.argv[0]))
    root = sys.argv[1]
    text = open(os.path.join(root, "itex/core/graph/native_layout/native_layout.cc")).read()
    gpu = text[text.index("GetCPUEigenNativeFormatInfo() {"):text.index("GetCPUNativeFormatInfo() {")]
    gpu = re.sub(r"//[^\n]*", "", gpu)
    entries = re.findall(r'\{\s*"([^"]+)"\s*,\s*"([^"]+)"\s*,\s*(\w+)\s*,\s*(\w+)\s*\}', gpu)
    table = [{"from": f, "to": t, "copy": c, "rule": r} for f, t, c, r in entries if "uantize" in f]
    with open(os.path.join(HERE, "rewrite_table.json"), "w") as f:
        json.dump(table, f, indent=1)
    print("%d quantized-op entries written" % len(table))


if __name__ == "__main__":
    main()
