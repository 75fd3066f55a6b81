"""Traces tests/frontend_models.py's models through the REFERENCE's core_v2 front end and records every stage.

    python tests/golden/make_frontend_golden.py [--reference <reference checkout>/ai-compiler-framework]

Needs the reference checkout and torch; no GPU. The reference's executor module imports `aicf_cuda._C` at
import time, which resolves to this repository's binding module (nothing is launched). Per model the JSON
keeps: the IR dump, the lowered list after stage A, after stage B, after stage C, after dtype-based selection
of the remaining ids (the order the reference's end-to-end test uses), the older opt_rules fusion followed by
kernel_select, the binding-plan dump, and the lowered dump text.
"""
from __future__ import annotations

import argparse
import os
import json
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REPO = HERE.parents[1]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", type=Path, default=Path(os.environ.get("AICF_REFERENCE_DIR") or HERE.parents[2] / "reference" / "ai-compiler-framework"))
    a = ap.parse_args()
    # The reference's python directory goes first: this repository ships an `aicf_fw.core_v2` import shim of its own
    # (both `aicf_fw` directories are namespace portions, so path order decides).
    sys.path[:0] = [str(a.reference / "python"), str(HERE.parent), str(REPO / "ai-compiler-framework_b200" / "python")]
    import torch
    from aicf_fw.core_v2 import dump_ir, dump_lowered, dump_plan, trace_ir
    from aicf_fw.core_v2 import ops as ref_ops
    from aicf_fw.core_v2.kernel_select import apply_kernel_selection
    from aicf_fw.core_v2.lower import lower_to_backend_ops
    from aicf_fw.core_v2.opt_rules import apply_opt_rules
    from aicf_fw.core_v2.plan import apply_kernel_decisions_stageB, build_binding_plan
    from aicf_fw.core_v2.rewrites.stageC_fuse_epilogue import stageC_fuse_gemm_epilogue
    from frontend_models import MODELS, build_model
    import aicf_fw.core_v2
    assert Path(aicf_fw.core_v2.__file__).resolve().is_relative_to(a.reference.resolve()), "wrong aicf_fw.core_v2 on the path"

    tdt = {"f16": torch.float16, "f32": torch.float32}
    out = {}
    for spec in MODELS:
        ir = trace_ir(lambda: build_model(ref_ops, spec, tdt[spec["dtype"]], torch.float32, torch.int32,
                                          device=torch.device("cuda:0")), name=spec["name"])
        a_ = lower_to_backend_ops(ir)
        b_ = apply_kernel_decisions_stageB(ir, a_)
        c_ = stageC_fuse_gemm_epilogue(ir, b_)
        # ids for the ops still without one, exactly as the reference's test fills them (kernel_select's table)
        sel = apply_kernel_selection(ir, c_)
        final = [dict(it, kernel_id=(it.get("kernel_id") or s.get("kernel_id"))) if (it.get("kernel_id") or s.get("kernel_id"))
                 else dict(it) for it, s in zip(c_, sel)]
        opt = apply_kernel_selection(ir, apply_opt_rules(ir, a_))
        out[spec["name"]] = {"ir_text": dump_ir(ir), "stage_a": a_, "stage_b": b_, "stage_c": c_, "final": final,
                             "opt_rules_then_select": opt, "plan_text": dump_plan(build_binding_plan(ir), name=spec["name"]),
                             "final_text": dump_lowered(final, name=spec["name"])}
    (HERE / "frontend_golden.json").write_text(json.dumps(out) + "\n")
    print(f"wrote {HERE / 'frontend_golden.json'}: {len(out)} models")


if __name__ == "__main__":
    main()
