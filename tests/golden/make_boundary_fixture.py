"""Turns the reference's committed boundary dumps into tests/golden/boundary_fixture.json.

    python tests/golden/make_boundary_fixture.py [--reference <reference checkout>/ai-compiler-framework]

Source: artifacts/20260128_222814_v2_kid_trace_by_id_test/{20_ir,30_lowered,40_plan,50_runtime_trace}.txt, the
output of the reference's own python_framework_test/v2_kid_trace_by_id_test.py (a 2-layer f16 MLP,
B=64, D=8, MSE + SGD). The JSON keeps exactly what those dumps pin: the lowered-op list with kernel
ids and attrs, the role/shape/dtype of every value, the runtime trace strings, the traced IR's node list,
and the three text dumps verbatim (they pin the printer's line formats).
"""
from __future__ import annotations

import argparse
import os
import ast
import json
import re
from pathlib import Path

HERE = Path(__file__).resolve().parent
ART = "artifacts/20260128_222814_v2_kid_trace_by_id_test"


def parse_lowered(text: str):
    ops = []
    pat = re.compile(r"#(\d+)\s+(\w+)\s+\(([^)]*)\)\s*->\s*\(([^)]*)\)\s*(\{[^}]*\})?\s*kid=(\S+)")
    for line in text.splitlines():
        m = pat.search(line)
        if not m:
            continue
        attrs = {}
        if m.group(5):
            for kv in m.group(5).strip("{}").split(","):
                k, v = kv.split("=")
                v = v.strip()
                attrs[k.strip()] = ast.literal_eval(v) if v in ("True", "False") or re.fullmatch(r"[-\d.e]+", v) else v
        ints = lambda s: [int(x) for x in s.split(",") if x.strip()]
        ops.append({"op": m.group(2), "inputs": ints(m.group(3)), "outputs": ints(m.group(4)), "attrs": attrs,
                    "kernel_id": m.group(6)})
    return ops


def parse_plan(text: str):
    vals = []
    pat = re.compile(r"v(\d+)\s+(\S+)\s+role=(\w+)\s+shape=\(([^)]*)\)\s+dtype=torch\.(\w+)")
    for line in text.splitlines():
        m = pat.search(line)
        if m:
            shape = [int(x) for x in m.group(4).split(",") if x.strip()]
            vals.append({"vid": int(m.group(1)), "name": m.group(2), "role": m.group(3), "shape": shape, "dtype": m.group(5)})
    return sorted(vals, key=lambda v: v["vid"])


def parse_ir_nodes(text: str):
    nodes = []
    pat = re.compile(r"#(\d+)\s+(\w+)\s+\(([^)]*)\)\s*->\s*\(([^)]*)\)(?:\s+\{(.*)\})?\s*$")
    vids = lambda s: [int(x.strip()[1:]) for x in s.split(",") if x.strip()]
    for line in text.split("[nodes]")[1].splitlines():
        m = pat.search(line)
        if not m:
            continue
        attrs = {}
        for kv in (m.group(5) or "").split(", "):
            if kv:
                k, v = kv.split("=", 1)
                attrs[k] = ast.literal_eval(v) if v in ("True", "False") or re.fullmatch(r"[-\d.e]+", v) else v
        nodes.append({"op": m.group(2), "inputs": vids(m.group(3)), "outputs": vids(m.group(4)), "attrs": attrs})
    return nodes


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", type=Path, default=Path(os.environ.get("AICF_REFERENCE_DIR") or HERE.parents[2] / "reference" / "ai-compiler-framework"))
    a = ap.parse_args()
    d = a.reference / ART
    fixture = {
        "source": f"{ART}/20_ir.txt, 30_lowered.txt, 40_plan.txt, 50_runtime_trace.txt",
        "ir_nodes": parse_ir_nodes((d / "20_ir.txt").read_text()),
        "text": {"ir": (d / "20_ir.txt").read_text(), "lowered": (d / "30_lowered.txt").read_text(),
                 "plan": (d / "40_plan.txt").read_text()},
        "lowered": parse_lowered((d / "30_lowered.txt").read_text()),
        "values": parse_plan((d / "40_plan.txt").read_text()),
        "runtime_trace": [l.strip() for l in (d / "50_runtime_trace.txt").read_text().splitlines() if l.strip()],
    }
    assert len(fixture["lowered"]) == 16 and len(fixture["values"]) == 18 and len(fixture["runtime_trace"]) == 16
    assert len(fixture["ir_nodes"]) == 12
    (HERE / "boundary_fixture.json").write_text(json.dumps(fixture, indent=1) + "\n")
    print(f"wrote {HERE / 'boundary_fixture.json'}")


if __name__ == "__main__":
    main()
