"""The reference's own unit-test suite (``tests/unit``, about a thousand tests), run unchanged against
this package aliased as ``nabla``.

Needs a checkout of the reference: set ``NABLA_REFERENCE_DIR`` to its root; without it the module is
skipped. The suite computes its expected values with jax, which this environment does not have, so
``tests/reference_harness`` provides a stand-in for the jax functions the suite calls, built on
``torch.func`` (the package under test never imports it), and a ``max.dtype`` module that hands out
this package's ``DType``.

Three items of the suite are expected to differ and are listed in ``EXPECTED_DIFFERENCES`` with the
reason; anything else that fails is a regression."""
import os
import re
import shutil
import subprocess
import sys
import textwrap

import pytest

REF = os.environ.get("NABLA_REFERENCE_DIR", "")
UNIT = os.path.join(REF, "tests", "unit") if REF else ""
REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HARNESS = os.path.join(REPO, "tests", "reference_harness")

pytestmark = pytest.mark.skipif(not (UNIT and os.path.isdir(UNIT)),
                                reason="NABLA_REFERENCE_DIR does not point at a reference checkout")

EXPECTED_DIFFERENCES = {
    # asserts that compiling a sharded function with dynamic dims raises NotImplementedError; it is supported here
    "tests/unit/test_compile.py::test_compile_sharded_dynamic",
    # asserts that reading the VJP of a conv on a (1, 1) mesh raises a device-mismatch ValueError; it works here
    "tests/unit/test_convolution.py::TestConvolution2D::test_conv2d_sharded_vjp_raises_current_device_mismatch",
    # a script that traces at import; its last scenario multiplies (4, 4) by (2, 4), which only a tracer that
    # never checks shapes lets through (shapes are checked when an op is recorded here)
    "tests/unit/test_partial_propagation.py",
}

CONFTEST = textwrap.dedent('''
    import importlib, pkgutil, sys
    sys.path[:0] = [{here!r}, {repo!r}, {harness!r}]
    import nabla_b200
    sys.modules["nabla"] = nabla_b200
    for m in pkgutil.walk_packages(nabla_b200.__path__, "nabla_b200."):
        if ".csrc" in m.name or ".lib" in m.name:
            continue
        try:
            sys.modules["nabla" + m.name[len("nabla_b200"):]] = importlib.import_module(m.name)
        except Exception:
            pass
''')


def test_reference_unit_suite_passes_against_this_package(tmp_path):
    shutil.copytree(UNIT, tmp_path / "tests" / "unit")
    (tmp_path / "tests" / "__init__.py").write_text("")
    (tmp_path / "conftest.py").write_text(CONFTEST.format(here=str(tmp_path), repo=REPO, harness=HARNESS))
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([str(tmp_path), REPO, HARNESS]))
    cmd = [sys.executable, "-m", "pytest", "tests/unit", "-q", "-p", "no:cacheprovider", "--continue-on-collection-errors",
           "-rfE", "--timeout", "900"]
    try:
        import xdist  # noqa: F401

        cmd += ["-n", str(min(8, os.cpu_count() or 1))]
    except ImportError:
        pass
    out = subprocess.run(cmd, cwd=tmp_path, env=env, capture_output=True, text=True, timeout=3600).stdout
    bad = set()
    for line in out.splitlines():
        m = re.match(r"^(FAILED|ERROR) (\S+)", line)
        if m:
            bad.add(m.group(2))
    summary = [ln for ln in out.splitlines() if " passed" in ln][-1:]
    passed = int(re.search(r"(\d+) passed", summary[0]).group(1)) if summary else 0
    unexpected = sorted(bad - EXPECTED_DIFFERENCES)
    assert not unexpected, "reference tests that fail against this package:\n" + "\n".join(unexpected) + "\n" + out[-3000:]
    assert passed >= 1000, f"only {passed} reference tests passed:\n{out[-3000:]}"


# stages of the reference's `Operation.__call__` that only make sense around a MAX graph under
# construction (attaching tangents to graph values, eager MAX execution, wrapping MAX values into
# tensors, checking MAX value types); the op call of this package has no such steps
NO_COUNTERPART = {"nabla_b200.ops.utils": {"adapt_and_reshard", "apply_jvp", "eager_execute", "package_outputs",
                                           "validate_physical_metadata"}}


def test_every_public_name_of_the_reference_package_exists_here():
    """Module by module: each public function, class and ``__all__`` entry of ``nabla/**.py`` is an
    attribute of the module of the same path under ``nabla_b200``."""
    import ast
    import importlib

    root = os.path.join(REF, "nabla")
    problems = []
    for dirpath, _, files in os.walk(root):
        for f in files:
            if not f.endswith(".py"):
                continue
            path = os.path.join(dirpath, f)
            rel = os.path.relpath(path, root)[:-3].replace(os.sep, ".")
            if rel.endswith("__init__"):
                rel = rel[:-len("__init__")].rstrip(".")
            name = "nabla_b200" + ("." + rel if rel else "")
            try:
                mod = importlib.import_module(name)
            except Exception as e:
                problems.append(f"{name}: cannot import ({e})")
                continue
            wanted = set()
            for node in ast.parse(open(path).read()).body:
                if isinstance(node, (ast.FunctionDef, ast.AsyncFunctionDef, ast.ClassDef)) and not node.name.startswith("_"):
                    wanted.add(node.name)
                elif isinstance(node, ast.Assign) and isinstance(node.value, (ast.List, ast.Tuple)):
                    if any(isinstance(t, ast.Name) and t.id == "__all__" for t in node.targets):
                        wanted |= {e.value for e in node.value.elts if isinstance(e, ast.Constant)}
            missing = sorted(n for n in wanted if not hasattr(mod, n) and n not in NO_COUNTERPART.get(name, ()))
            if missing:
                problems.append(f"{name}: {missing}")
    assert not problems, "\n".join(problems)
