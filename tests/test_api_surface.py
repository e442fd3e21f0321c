"""Names and signatures of the reference's Python surface (common.py, gpi.py, GaspiEx.py,
ComprEx.py, allreduce.py, allreduceOp.py, keras/callbacks.py, keras/comprex_optimizer.py) against
this package: every public class, every public method, every parameter name of the reference must
exist here (extra parameters with defaults are allowed).  The reference's files are only parsed
(``ast``), never imported.  Needs ``COMPREX_REFERENCE``; skipped without it."""
import ast
import inspect
import os

import pytest

import comprex_b200 as cx
from comprex_b200 import allreduceOp, callbacks, common, gpi, optim

REF = os.environ.get("COMPREX_REFERENCE")
pytestmark = pytest.mark.skipif(not REF or not os.path.exists(os.path.join(REF or "", "allreduce.py")),
                                reason="COMPREX_REFERENCE does not point at the reference's tree")

MODULES = {"common.py": common, "gpi.py": gpi, "GaspiEx.py": cx, "ComprEx.py": cx, "allreduce.py": cx,
           "allreduceOp.py": allreduceOp, "keras/callbacks.py": callbacks, "keras/comprex_optimizer.py": optim}
# reference names with another spelling here, and internals of the reference's ctypes/TF plumbing
RENAMED = {"Getable": "Gettable"}
SKIP_CLASSES = set()
SKIP_METHODS = {"_resource_apply_dense", "_resource_apply_sparse", "_create_slots", "_prepare_local",
                "get_config", "_aggregate_gradients", "_create_hypers", "_prepare"}


def reference_surface(path):
    tree = ast.parse(open(path).read())
    out = {}
    for node in tree.body:
        if isinstance(node, ast.ClassDef):
            methods = {}
            for item in node.body:
                if isinstance(item, ast.FunctionDef) and (not item.name.startswith("_") or item.name == "__init__"):
                    methods[item.name] = [a.arg for a in item.args.args if a.arg != "self"]
            out[node.name] = methods
        elif isinstance(node, ast.FunctionDef) and not node.name.startswith("_"):
            out[node.name] = [a.arg for a in node.args.args]
    return out


@pytest.mark.parametrize("rel", sorted(MODULES))
def test_reference_names_and_parameters_exist(rel):
    mod = MODULES[rel]
    missing = []
    for name, body in reference_surface(os.path.join(REF, rel)).items():
        if name in SKIP_CLASSES:
            continue
        mine = getattr(mod, RENAMED.get(name, name), None) or getattr(cx, RENAMED.get(name, name), None)
        if mine is None:
            missing.append(name)
            continue
        if isinstance(body, list):                         # module-level function
            have = inspect.signature(mine).parameters
            missing += [f"{name}({a})" for a in body if a not in have]
            continue
        for meth, args in body.items():
            if meth in SKIP_METHODS:
                continue
            fn = getattr(mine, meth, None)
            if fn is None:
                missing.append(f"{name}.{meth}")
                continue
            params = inspect.signature(fn).parameters
            flexible = any(p.kind in (p.VAR_POSITIONAL, p.VAR_KEYWORD) for p in params.values())
            if not flexible:
                missing += [f"{name}.{meth}({a})" for a in args if a not in params]
    assert not missing, "missing from this package: " + ", ".join(missing)
