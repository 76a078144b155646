#!/usr/bin/env python
"""Writes tests/golden/kernel_table_v1.json: the member list of the reference's
`KernelTableV1` (index, name, C argument list), parsed from
packs/cuda/src/abi.cuh of a truespar/paddock checkout.

    python tests/golden/gen_kernel_table.py /path/to/paddock

tests/test_pack_abi.py holds every PDK_SLOT_* index of include/paddock_pack.h and
the argument count of every served slot against this list, so that a slot added
with an off-by-one index cannot pass.  oracle/build_ref.sh reruns this script
whenever it finds the checkout."""
import json
import os
import re
import sys


def parse(abi_cuh):
    src = open(abi_cuh).read()
    i = src.index("struct KernelTableV1 {")
    depth, j = 0, i
    for p in range(src.index("{", i), len(src)):       # the struct's own closing brace
        if src[p] == "{":
            depth += 1
        elif src[p] == "}":
            depth -= 1
            if depth == 0:
                j = p
                break
    body = src[i:j]
    body = re.sub(r"//[^\n]*", "", body)
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    decls = [" ".join(d.split()) for d in body.split(";")]
    decls = [d for d in decls if "(*" in d]             # every function-pointer member, whatever it returns
    out = []
    for k, d in enumerate(decls):
        m = re.search(r"\(\*\s*(\w+)\s*\)\s*\((.*)\)$", d)
        out.append([k, m.group(1), m.group(2)])
    return out


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("PADDOCK_REFERENCE", "")
    path = os.path.join(ref, "packs", "cuda", "src", "abi.cuh")
    if not os.path.exists(path):
        raise SystemExit(f"no packs/cuda/src/abi.cuh under {ref!r}")
    table = parse(path)
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "kernel_table_v1.json")
    with open(out, "w") as f:
        json.dump({"source": "packs/cuda/src/abi.cuh, struct KernelTableV1", "members": table}, f, separators=(",", ":"))
    print(f"{len(table)} members -> {out}")


if __name__ == "__main__":
    main()
