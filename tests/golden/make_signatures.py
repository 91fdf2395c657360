"""Write ``operator_signatures.json``: the Python signatures of the reference's operators on this path.

    OASR_REFERENCE=<path of the reference checkout> python tests/golden/make_signatures.py

Imports the reference package (torch backend) and records, for every name ``oasr_b200.install`` rebinds,
the parameter list of ``oasr.<name>`` (``oasr.functionals.attention.<name>`` for the attention calls):
name, kind and default of every parameter, in order.  ``tests/test_install.py`` holds this package's
operators to that snapshot.
"""
from __future__ import annotations

import inspect
import json
import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))
REF = os.environ.get("OASR_REFERENCE")
if not REF:
    raise SystemExit("set OASR_REFERENCE to the path of the reference checkout")
os.environ["OASR_LAYERS_BACKEND"] = "torch"
sys.path.insert(0, REF)

import oasr  # noqa: E402  (the reference)
import oasr.functionals.attention as ref_attention  # noqa: E402

import oasr_b200  # noqa: E402


def describe(fn):
    out = []
    for p in inspect.signature(fn).parameters.values():
        default = None if p.default is inspect.Parameter.empty else repr(p.default)
        out.append({"name": p.name, "kind": p.kind.name, "default": default})
    return out


snapshot = {}
for name in oasr_b200.OPERATOR_NAMES:
    snapshot[name] = describe(getattr(oasr, name))
for name in ("fmha", "fmha_varlen"):
    snapshot[name] = describe(getattr(ref_attention, name))
(HERE / "operator_signatures.json").write_text(json.dumps(snapshot, indent=1, sort_keys=True) + "\n")
print(f"{len(snapshot)} signatures written")
