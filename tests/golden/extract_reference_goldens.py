"""Extracts the golden output vectors of the reference's own graph tests into a JSON fixture.

Run in a container that has the reference checked out:

    python tests/golden/extract_reference_goldens.py <path of the reference checkout>

It reads ``tests/vulkan.cpp`` as text, finds the expected-output array literal of each listed
gtest case and writes ``tests/golden/reference_goldens.json``.  Only numbers are taken; the
inputs of each case are simple fills (iota, ones) restated in ``tests/test_oracle_golden.py``
with the line they come from.
"""
from __future__ import annotations

import json
import os
import re
import sys

# gtest case -> (name of the expected array in the case body, element type, shape)
CASES = {
    "MaxPool2D": ("ref", "int8", [1, 8, 8, 3]),
    "TwoLayerMaxPool2D": ("ref", "int8", [1, 4, 4, 3]),
    "Conv2D": ("ref", "int32", [1, 4, 4, 3]),
    "Conv2DAccumulatorInt64": ("expectedValues", "int64", [1, 2, 2, 4]),
    "Concat": ("ref", "int8", [1, 4, 2, 2]),
    "ConcatMultipleDispatchesPreserveInputLiveRange": ("expected", "float32", [12]),
    "Slice": ("ref", "int8", [1, 2, 2, 2]),
    "NOPOutputs": ("ref", "int8", [1, 2, 2, 2]),
    "GraphConstantARM": ("ref", "int8", [5]),
    "HigherRankConstant": ("ref", "int8", [1, 3, 3, 1]),
    "Maximum": ("ref", "int32", [1, 2, 2, 2]),
    "Conv3DLargeStridePadRegression": ("expectedValues", "int32", [1, 3, 2, 2, 3]),
}

# further arrays of a case that its inputs are built from: fixture name -> (gtest case, array, type, shape)
EXTRA = {
    "Conv3DLargeStridePadRegression.relevantWeights": ("Conv3DLargeStridePadRegression", "relevantWeights", "int8",
                                                       [96]),
}

_WIDTH = {"int8": 8, "int32": 32, "int64": 64}


def _case_body(text: str, name: str) -> tuple[str, int]:
    m = re.search(r"TEST\(MLEmulationLayerForVulkan,\s*%s\)\s*\{" % re.escape(name), text)
    if not m:
        raise KeyError(name)
    nxt = re.search(r"\nTEST\(", text[m.end():])
    end = m.end() + (nxt.start() if nxt else len(text) - m.end())
    return text[m.start():end], text[:m.start()].count("\n") + 1


def _array_literal(body: str, var: str) -> str:
    m = re.search(r"\b%s\b(?:\[[^\]]*\])*\s*(?:=\s*)?\{" % re.escape(var), body)
    if not m:
        raise KeyError(var)
    depth, i = 1, m.end()
    while depth:
        depth += {"{": 1, "}": -1}.get(body[i], 0)
        i += 1
    return body[m.end():i - 1]


def _numbers(literal: str, dtype: str):
    literal = re.sub(r"//[^\n]*", "", literal)
    toks = re.findall(r"-?0x[0-9a-fA-F]+|-?\d+(?:\.\d+)?", literal)
    out = []
    for t in toks:
        if dtype == "float32":
            out.append(float(t))
            continue
        v = int(t, 0)
        bits = _WIDTH[dtype]
        if v >= 1 << (bits - 1):  # literals are written as unsigned bytes/words
            v -= 1 << bits
        out.append(v)
    return out


def main(ref_root: str) -> None:
    src = os.path.join(ref_root, "tests", "vulkan.cpp")
    text = open(src, encoding="utf-8").read()
    goldens = {}
    for name, (var, dtype, shape) in CASES.items():
        body, line = _case_body(text, name)
        values = _numbers(_array_literal(body, var), dtype)
        goldens[name] = {
            "source": "tests/vulkan.cpp:%d" % line,
            "dtype": dtype,
            "shape": shape if shape is not None else [len(values)],
            "values": values,
        }
    for name, (case, var, dtype, shape) in EXTRA.items():
        body, line = _case_body(text, case)
        goldens[name] = {
            "source": "tests/vulkan.cpp:%d" % line,
            "dtype": dtype,
            "shape": shape,
            "values": _numbers(_array_literal(body, var), dtype),
        }
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_goldens.json")
    with open(dst, "w", encoding="utf-8") as f:
        json.dump(goldens, f, indent=1)
    print("wrote", dst, {k: len(v["values"]) for k, v in goldens.items()})


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MLEL_REFERENCE_ROOT", "/root/reference"))
