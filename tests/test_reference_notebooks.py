"""The reference's example notebooks, executed unchanged against this package aliased as ``nabla``.

Needs a checkout of the reference: set ``NABLA_REFERENCE_DIR`` to its root (the directory that holds
``examples/*.ipynb``); without it the module is skipped. Notebook 12 builds Mojo kernels through the
MAX toolchain and is not applicable (custom kernels here are CUDA sources, ``ops/custom.py``)."""
import glob
import importlib
import json
import os
import pkgutil
import sys

import pytest

REF = os.environ.get("NABLA_REFERENCE_DIR", "")
NOTEBOOKS = sorted(glob.glob(os.path.join(REF, "examples", "*.ipynb"))) if REF else []
NOT_APPLICABLE = ("12_custom_mojo_kernels",)

pytestmark = pytest.mark.skipif(not NOTEBOOKS, reason="NABLA_REFERENCE_DIR does not point at a reference checkout")


@pytest.fixture(scope="module")
def nabla_alias():
    """``import nabla`` and ``from nabla.x.y import z`` resolve to this package for the duration."""
    import nabla_b200

    added = []
    names = ["nabla_b200"] + [m.name for m in pkgutil.walk_packages(nabla_b200.__path__, "nabla_b200.")
                              if ".csrc" not in m.name and ".lib" not in m.name]
    for name in names:
        try:
            mod = importlib.import_module(name)
        except Exception:
            continue
        alias = "nabla" + name[len("nabla_b200"):]
        if alias not in sys.modules:
            sys.modules[alias] = mod
            added.append(alias)
    yield
    for alias in added:
        sys.modules.pop(alias, None)


@pytest.mark.parametrize("path", NOTEBOOKS, ids=[os.path.basename(p)[:-6] for p in NOTEBOOKS])
def test_reference_notebook_runs_unchanged(path, nabla_alias):
    if any(tag in path for tag in NOT_APPLICABLE):
        pytest.skip("depends on the MAX / Mojo toolchain")
    with open(path) as f:
        cells = json.load(f)["cells"]
    scope = {"__name__": "__main__"}
    for i, cell in enumerate(cells):
        if cell["cell_type"] != "code":
            continue
        src = "\n".join(line for line in "".join(cell["source"]).splitlines() if not line.strip().startswith(("%", "!")))
        if src.strip():
            exec(compile(src, f"{os.path.basename(path)}[cell {i}]", "exec"), scope)
