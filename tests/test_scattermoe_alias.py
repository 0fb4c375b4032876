"""`import scattermoe` resolves to this package: the names the reference exports (scattermoe/__init__.py:1-15) and
every import its own test file makes (tests/test_mlp.py:1-8)."""
import ast
import importlib
import os

import pytest


def test_alias_package_binds_every_reference_module_name():
    import scattermoe
    import scattermoe_b200
    assert scattermoe.__all__ == ["flatten_sort_count", "parallel_linear", "ParallelExperts", "parallel_experts",
                                  "kernels", "mlp", "utils"]
    for sub in ("parallel_experts", "kernels", "kernels.ops", "kernels.single", "mlp", "utils", "utils.replace_moe"):
        assert importlib.import_module("scattermoe." + sub) is importlib.import_module("scattermoe_b200." + sub)
    from scattermoe.mlp import MLP, GLUMLP
    assert MLP is scattermoe_b200.mlp.MLP and GLUMLP is scattermoe_b200.mlp.GLUMLP
    # module globals are read at call time, so the reference test's switch reaches the implementation (ops.py:7)
    saved = scattermoe_b200.kernels.ops.ALLOW_TF32
    try:
        scattermoe.kernels.ops.ALLOW_TF32 = False
        assert scattermoe_b200.kernels.ops.ALLOW_TF32 is False
    finally:
        scattermoe_b200.kernels.ops.ALLOW_TF32 = saved
    assert scattermoe.kernels.ops.BLOCK_M == 128


def test_imports_of_the_reference_test_file_resolve():
    path = "/root/reference/tests/test_mlp.py"
    if not os.path.isfile(path):
        pytest.skip("no reference checkout on this machine")
    tree = ast.parse(open(path).read())
    seen = 0
    for node in ast.walk(tree):
        if isinstance(node, ast.ImportFrom) and node.module and node.module.split(".")[0] == "scattermoe":
            mod = importlib.import_module(node.module)
            for a in node.names:
                assert hasattr(mod, a.name), (node.module, a.name)
                seen += 1
        elif isinstance(node, ast.Import):
            for a in node.names:
                if a.name.split(".")[0] == "scattermoe":
                    importlib.import_module(a.name)
                    seen += 1
        elif isinstance(node, ast.Attribute):
            # attribute chains rooted at the package, e.g. scattermoe.kernels.ops.ALLOW_TF32
            chain, cur = [node.attr], node.value
            while isinstance(cur, ast.Attribute):
                chain.append(cur.attr)
                cur = cur.value
            if isinstance(cur, ast.Name) and cur.id == "scattermoe":
                obj = importlib.import_module("scattermoe")
                for part in reversed(chain):
                    assert hasattr(obj, part), ".".join(reversed(chain))
                    obj = getattr(obj, part)
                seen += 1
    assert seen >= 3
