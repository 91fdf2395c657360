"""CPU: the drop-in boundary.  ``oasr_b200.install(oasr)`` rebinds exactly the reference's operator names, hands back
what restores them, and every operator keeps the reference's Python signature.

The reference's layers look operators up as attributes of the ``oasr`` package at call time (``oasr.gemm(...)``,
oasr/layers/linear.py:103; ``from oasr.functionals.attention import fmha`` inside the call,
oasr/layers/attention/attention.py:266) and its own shape recorder patches the same attributes
(oasr/tune/capture.py:23-26), so rebinding them is the whole integration."""
import inspect
import json
import types
from pathlib import Path

import oasr_b200

SNAPSHOT = json.loads((Path(__file__).resolve().parent / "golden" / "operator_signatures.json").read_text())
ATTENTION = ("fmha", "fmha_varlen")


def _stub_package():
    """A module tree shaped like the reference package: flat operator attributes plus functionals.attention."""
    pkg = types.ModuleType("oasr_stub")
    pkg.functionals = types.ModuleType("oasr_stub.functionals")
    pkg.functionals.attention = types.ModuleType("oasr_stub.functionals.attention")
    originals = {}
    for name in oasr_b200.OPERATOR_NAMES + ATTENTION:
        fn = (lambda n: (lambda *a, **k: n))(name)
        originals[name] = fn
        setattr(pkg, name, fn)
    for name in ATTENTION:
        setattr(pkg.functionals.attention, name, originals[name])
    pkg.untouched = object()
    pkg.greedy_search = lambda *a, **k: "decoder"       # a name outside the hot path
    return pkg, originals


def test_install_rebinds_exactly_the_operator_names_and_returns_what_restores_them():
    pkg, originals = _stub_package()
    before = dict(vars(pkg))
    saved = oasr_b200.install(pkg)
    expected = set(oasr_b200.OPERATOR_NAMES) | set(ATTENTION)
    assert set(SNAPSHOT) == expected
    changed = {k for k in before if vars(pkg)[k] is not before[k]}
    assert changed == expected                                           # nothing else on the package was touched
    for name in expected:
        assert getattr(pkg, name) is getattr(oasr_b200, name)
    for name in ATTENTION:
        assert getattr(pkg.functionals.attention, name) is getattr(oasr_b200, name)
    assert set(saved) == expected | {"functionals.attention." + n for n in ATTENTION}
    for name in expected:
        assert saved[name] is originals[name]
    # restoring
    oasr_b200.uninstall(pkg, saved)
    for name in expected:
        assert getattr(pkg, name) is originals[name]
    for name in ATTENTION:
        assert getattr(pkg.functionals.attention, name) is originals[name]
    assert pkg.greedy_search() == "decoder"


def test_operator_signatures_equal_the_reference_snapshot():
    """Same parameter names, order, kinds and defaults; this package may only ADD keyword-only parameters with
    defaults (extensions such as ``out_dtype`` of gemm_log_softmax)."""
    supersets = []
    for name, ref_params in SNAPSHOT.items():
        own = list(inspect.signature(getattr(oasr_b200, name)).parameters.values())
        own_by_name = {p.name: p for p in own}
        for rp in ref_params:
            assert rp["name"] in own_by_name, f"{name}: parameter {rp['name']} is missing"
            p = own_by_name[rp["name"]]
            assert p.kind.name == rp["kind"], f"{name}.{p.name}: kind {p.kind.name} != {rp['kind']}"
            default = None if p.default is inspect.Parameter.empty else repr(p.default)
            assert default == rp["default"], f"{name}.{p.name}: default {default} != {rp['default']}"
        # positional order of the shared parameters
        ref_pos = [rp["name"] for rp in ref_params if rp["kind"] != "KEYWORD_ONLY"]
        own_pos = [p.name for p in own if p.kind.name != "KEYWORD_ONLY"]
        assert own_pos == ref_pos, f"{name}: positional parameters {own_pos} != {ref_pos}"
        extra = [p for p in own if p.name not in {rp["name"] for rp in ref_params}]
        for p in extra:
            assert p.kind.name == "KEYWORD_ONLY" and p.default is not inspect.Parameter.empty, f"{name}: extra parameter {p.name}"
        if extra:
            supersets.append(name)
    print("keyword-only supersets of the reference signature:", supersets)
