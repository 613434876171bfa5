"""Extracts the literal tensors of the reference's own CPU tests into reference_vectors.json.

Run where the reference tree is present:
    python tests/golden/extract_reference_vectors.py <reference checkout>

Every `TEST(Suite, Name)` body of the listed files is scanned for
`Tensor X(dtype, {shape}); X.initialize({...});` pairs; the nested initialiser lists are stored
as flat value lists with their shape and dtype. What each test does with its tensors (which
operation, which tensor is the expectation) is written down by hand in tests/test_reference_vectors.py,
next to the file:line of the test it mirrors.
"""
import ast
import json
import re
import sys
from pathlib import Path

FILES = ["tests/cpu/test-matmul.cpp", "tests/cpu/test-operations.cpp", "tests/cpu/test-reductions.cpp",
         "tests/cpu/test-convolutions.cpp", "tests/cpu/test-functions.cpp", "tests/cpu/test-non-contiguous.cpp"]


def balanced(text, start, open_ch, close_ch):
    depth = 0
    for i in range(start, len(text)):
        if text[i] == open_ch:
            depth += 1
        elif text[i] == close_ch:
            depth -= 1
            if depth == 0:
                return i
    raise ValueError("unbalanced")


def flatten(v, out):
    if isinstance(v, (list, tuple)):
        for x in v:
            flatten(x, out)
    else:
        out.append(v)


def main(root):
    root = Path(root)
    result = {}
    for rel in FILES:
        path = root / rel
        if not path.exists():
            continue
        text = path.read_text()
        for m in re.finditer(r"TEST\(\s*(\w+)\s*,\s*(\w+)\s*\)\s*\{", text):
            end = balanced(text, m.end() - 1, "{", "}")
            body = text[m.end():end]
            line = text.count("\n", 0, m.start()) + 1
            tensors = {}
            for t in re.finditer(r"Tensor\s+(\w+)\s*\(\s*(\w+)\s*,\s*\{([^}]*)\}\s*\)\s*;", body):
                name, dtype, shape = t.group(1), t.group(2), [int(x) for x in t.group(3).split(",") if x.strip()]
                init = re.search(r"\b" + name + r"\.initialize\(", body[t.end():])
                if not init:
                    continue
                s = t.end() + init.end() - 1
                e = balanced(body, s, "(", ")")
                raw = re.sub(r"//[^\n]*", "", body[s + 1:e])
                raw = raw.replace("{", "[").replace("}", "]")
                raw = re.sub(r"(?<=[0-9.])f\b", "", raw)
                try:
                    values = []
                    flatten(ast.literal_eval(raw.strip()), values)
                except Exception:
                    continue
                n = 1
                for d in shape:
                    n *= d
                if len(values) != n:
                    continue
                tensors[name] = {"dtype": dtype, "shape": shape, "values": values}
            # `Tensor X = {{...}, {...}};`: dtype and shape follow from the literal (float32 / int32)
            for t in re.finditer(r"Tensor\s+(\w+)\s*=\s*\{", body):
                s = t.end() - 1
                e = balanced(body, s, "{", "}")
                raw = re.sub(r"//[^\n]*", "", body[s:e + 1]).replace("{", "[").replace("}", "]")
                is_float = bool(re.search(r"[0-9.]f\b|\d\.\d", raw))
                raw = re.sub(r"(?<=[0-9.])f\b", "", raw)
                try:
                    nested = ast.literal_eval(raw.strip())
                except Exception:
                    continue
                shape, probe = [], nested
                while isinstance(probe, list):
                    shape.append(len(probe))
                    probe = probe[0]
                values = []
                flatten(nested, values)
                tensors[t.group(1)] = {"dtype": "float32" if is_float else "int32", "shape": shape, "values": values}
            # element-wise expectations: ASSERT_EQ(Z[i][j], value)
            asserts = []
            for a in re.finditer(r"(?:ASSERT|EXPECT)_(?:EQ|FLOAT_EQ|NEAR)\(\s*(\w+)((?:\[\d+\])+)\s*,\s*(-?[0-9.]+(?:e-?\d+)?)f?\s*[,)]", body):
                index = [int(x) for x in re.findall(r"\[(\d+)\]", a.group(2))]
                asserts.append([a.group(1), index, float(a.group(3))])
            if tensors:
                entry = {"source": f"{rel}:{line}", "tensors": tensors}
                if asserts:
                    entry["asserts"] = asserts
                result[f"{m.group(1)}.{m.group(2)}"] = entry
    out = Path(__file__).resolve().parent / "reference_vectors.json"
    out.write_text(json.dumps(result, indent=0, separators=(",", ":")))
    print(f"{len(result)} tests, {sum(len(v['tensors']) for v in result.values())} tensors -> {out}")
    for k, v in result.items():
        print(k, v["source"], {n: t["shape"] for n, t in v["tensors"].items()})


if __name__ == "__main__":
    import os
    where = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("TANNIC_REFERENCE")
    if not where:
        sys.exit("usage: extract_reference_vectors.py <reference source tree>  (or set TANNIC_REFERENCE)")
    main(where)
