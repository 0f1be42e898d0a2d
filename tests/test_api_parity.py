"""Public signatures against the reference's source, read as text (no import, so no Triton
and no GPU needed): every optimizer constructor, ``cast_model``, ``enable_gradient_release``
and the tensor functions take the same arguments with the same defaults, and the package
exports the same names."""

import ast
import inspect
import os

import pytest

import flashoptim_b200 as fo

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref", "flashoptim")

pytestmark = pytest.mark.skipif(not os.path.exists(os.path.join(REF, "optimizers.py")),
                                reason="reference library is not installed under baseline/_ref")


def _ref_functions():
    tree = ast.parse(open(os.path.join(REF, "optimizers.py")).read())
    out = {}
    for node in tree.body:
        if isinstance(node, ast.FunctionDef):
            out[node.name] = node
        elif isinstance(node, ast.ClassDef):
            for item in node.body:
                if isinstance(item, ast.FunctionDef) and item.name == "__init__":
                    out[node.name] = item
    return out


def _ref_signature(fn: ast.FunctionDef):
    args = fn.args
    names = [a.arg for a in args.posonlyargs + args.args]
    defaults = [None] * (len(names) - len(args.defaults)) + [ast.literal_eval(d) if _literal(d) else ast.unparse(d)
                                                             for d in args.defaults]
    sig = list(zip(names, defaults))
    for a, d in zip(args.kwonlyargs, args.kw_defaults):
        sig.append((a.arg, None if d is None else (ast.literal_eval(d) if _literal(d) else ast.unparse(d))))
    return [(n, d) for n, d in sig if n != "self"]


def _literal(node) -> bool:
    try:
        ast.literal_eval(node)
        return True
    except Exception:
        return False


def _our_signature(obj):
    target = obj.__init__ if inspect.isclass(obj) else obj
    sig = []
    for name, p in inspect.signature(target).parameters.items():
        if name == "self":
            continue
        default = None if p.default is inspect.Parameter.empty else p.default
        sig.append((name, default))
    return sig


@pytest.mark.parametrize("name", [
    "FlashAdam", "FlashAdamW", "FlashLion", "FlashSGD", "FlashSGDW", "cast_model", "enable_gradient_release",
    "quantize", "dequantize", "compute_ecc_bits", "reconstruct_fp32_param",
])
def test_signature_matches_the_reference(name):
    ref = _ref_functions()[name]
    theirs = _ref_signature(ref)
    ours = _our_signature(getattr(fo, name))
    assert [n for n, _ in ours] == [n for n, _ in theirs]
    for (n, mine), (_, want) in zip(ours, theirs):
        if isinstance(want, str) and not isinstance(mine, str):
            # a default spelled as an expression in the reference (e.g. torch.bfloat16, GROUP_SIZE)
            assert want.split(".")[-1] in repr(mine) or str(mine) in want or want.isupper(), (n, mine, want)
        elif isinstance(want, (int, float)) and not isinstance(want, bool):
            assert mine == pytest.approx(want), (n, mine, want)
        else:
            assert mine == want, (n, mine, want)


def test_package_exports_every_name_of_the_reference():
    tree = ast.parse(open(os.path.join(REF, "__init__.py")).read())
    names = None
    for node in tree.body:
        if isinstance(node, ast.Assign) and any(getattr(t, "id", "") == "__all__" for t in node.targets):
            names = ast.literal_eval(node.value)
    assert names and set(names) <= set(fo.__all__)
    assert all(hasattr(fo, n) for n in names)


def test_optimizer_base_class_has_every_public_method_of_the_reference():
    tree = ast.parse(open(os.path.join(REF, "optimizers.py")).read())
    for node in tree.body:
        if isinstance(node, ast.ClassDef) and node.name == "FlashOptimizer":
            methods = [i for i in node.body if isinstance(i, ast.FunctionDef) and not i.name.startswith("_")]
            break
    assert len(methods) >= 6
    for m in methods:
        ours = getattr(fo.FlashOptimizer, m.name, None)
        assert callable(ours), m.name
        want = [a.arg for a in m.args.args if a.arg != "self"]
        have = [n for n in inspect.signature(ours).parameters if n != "self"]
        assert have[:len(want)] == want, (m.name, have, want)


def test_gradient_release_handle_has_the_reference_members():
    tree = ast.parse(open(os.path.join(REF, "optimizers.py")).read())
    for node in tree.body:
        if isinstance(node, ast.ClassDef) and node.name == "GradientReleaseHandle":
            members = {i.name for i in node.body if isinstance(i, ast.FunctionDef) and not i.name.startswith("_")}
    assert members and all(hasattr(fo.GradientReleaseHandle, m) for m in members), members
