"""Extracts the op definitions of the hot-path ops from the reference's registration code into tests/golden/op_defs.json.

The reference registers its own ops (the `_ITEX*` and `Fp8*` names TensorFlow does not know) through
TF_NewOpDefinitionBuilder / TF_OpDefinitionBuilderAddInput / AddOutput / AddAttr (itex/core/ops/nn_ops.cc,
itex/core/ops/fp8_ops.cc).  The argument strings of those calls ARE the interface a drop-in plugin has to register
verbatim, so the fixture holds exactly them, per op name, for the names this library implements.

Run where the reference checkout is available:
    python tests/golden/make_opdef_fixture.py /path/to/reference
"""
import json
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
FILES = ("itex/core/ops/nn_ops.cc", "itex/core/ops/fp8_ops.cc")
CALL = re.compile(r'TF_OpDefinitionBuilder(AddInput|AddOutput|AddAttr)\(\s*\w+\s*,((?:\s*"(?:[^"\\]|\\.)*")+)\s*\)', re.S)
LIT = re.compile(r'"((?:[^"\\]|\\.)*)"')


def extract(root):
    defs = {}
    for rel in FILES:
        text = open(os.path.join(root, rel)).read()
        starts = [(m.start(), m.group(1)) for m in re.finditer(r'TF_NewOpDefinitionBuilder\(\s*"([^"]+)"\s*\)', text)]
        for (pos, name), nxt in zip(starts, [s[0] for s in starts[1:]] + [len(text)]):
            end = text.find("TF_RegisterOpDefinition", pos)
            body = text[pos:min(end if end >= 0 else nxt, nxt)]
            d = {"inputs": [], "outputs": [], "attrs": [], "source": rel}
            for kind, lits in CALL.findall(body):
                spec = "".join(LIT.findall(lits))
                d[{"AddInput": "inputs", "AddOutput": "outputs", "AddAttr": "attrs"}[kind]].append(spec)
            defs[name] = d
    return defs


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: %s /path/to/reference-checkout" % os.path.basename(sys.argv[0]))
    root = sys.argv[1]
    wanted = json.load(open(os.path.join(HERE, "op_names.json")))
    defs = extract(root)
    out = {n: defs[n] for n in wanted if n in defs}
    missing = [n for n in wanted if n not in defs]
    with open(os.path.join(HERE, "op_defs.json"), "w") as f:
        json.dump({"ops": out, "defined_by_tensorflow": missing}, f, indent=1, sort_keys=True)
    print("%d op definitions written; %d names are TensorFlow's own ops" % (len(out), len(missing)))


if __name__ == "__main__":
    main()
