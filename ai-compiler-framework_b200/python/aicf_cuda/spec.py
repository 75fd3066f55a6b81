"""Value table of a plan: roles, naming rules and the ValueSpec record. Pure Python: this module (and
`lowering.py`, which needs nothing else) can be imported on a machine without the CUDA library."""
from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Optional, Tuple

ROLE_INPUT, ROLE_PARAM, ROLE_STATIC = 0, 1, 2

_PARAM_RE = re.compile(r"^\d+\.(W|b)$")


def classify_role(name: str) -> int:
    """Role of a value from its name, as the reference's binding plan decides it:
    'x' / 't' (and 'labels' for the cross-entropy graphs) are inputs, '<n>.W' / '<n>.b' are
    parameters, everything else is a plan-owned static."""
    if name in ("x", "t", "labels"):
        return ROLE_INPUT
    if _PARAM_RE.match(name):
        return ROLE_PARAM
    return ROLE_STATIC


def needs_zero_init(name: str) -> bool:
    return name.startswith("opt.step") or name.startswith("opt.m.") or name.startswith("opt.v.")


@dataclass
class ValueSpec:
    vid: int
    name: str
    shape: Tuple[int, ...]
    dtype: str
    role: Optional[int] = None        # None -> classify_role(name)
    persistent: bool = False          # keep out of arena reuse (read after the step)
    zero_init: Optional[bool] = None  # None -> needs_zero_init(name)
    alias_of: Optional[int] = None
    peer_visible: bool = False        # mapped by the other data-parallel ranks (gradients, broadcast copies)
