"""Writes tests/golden/ffi_signatures.json: name, argument names/types and return type of every
`extern "C"` function the reference declares in core/src/cuda_ffi.rs, as plain data.

    python tests/golden/make_ffi_signatures.py <path to the reference checkout>

tests/test_abi.py compares include/nlh_ffi.h against this file, so the drop-in prototypes are
checked against the reference's declarations wherever the tests run.
"""
import json
import os
import re
import sys


def parse(path):
    text = open(os.path.join(path, "core", "src", "cuda_ffi.rs")).read()
    text = re.sub(r"//[^\n]*", "", text)
    out = {}
    for m in re.finditer(r"fn (\w+)\s*\((.*?)\)\s*(?:->\s*([\w:]+))?\s*;", text, flags=re.S):
        args = [a.strip() for a in m.group(2).split(",") if a.strip()]
        out[m.group(1)] = {"args": [[a.split(":")[0].strip(), " ".join(a.split(":", 1)[1].split())] for a in args],
                           "ret": m.group(3)}
    return out


if __name__ == "__main__":
    sigs = parse(sys.argv[1])
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ffi_signatures.json")
    json.dump(sigs, open(dst, "w"), indent=0, sort_keys=True)
    print(dst, len(sigs), "functions")
