"""Runs the reference's own hook tests against this package's patcher modules.

The reference's ``tests/patcher/test_patcher_mmcv.py`` loads ``mx_driving/patcher/*.py``
straight from files under its project root. When ``MSDA_REFERENCE_ROOT`` names a checkout of
the reference, this test lays this package's patcher modules at those paths inside a
temporary tree, copies that one test file next to them (nothing is copied into this
repository) and runs, in a child process, the test classes of the patches this package
implements: MultiScaleDeformableAttention, DeformConv, ModulatedDeformConv and the Patcher
integration class (tests/patcher/test_patcher_mmcv.py:85-202, 288-314). The reference's
module also defines sparse-convolution, stream and DDP patches; the test file reads those
names at import time, so the temporary ``mmcv_patch.py`` re-exports this package's module and
sets the three absent names to ``None`` — their test classes are not selected.
Skipped when the variable is unset (the reference is not available on every machine).
"""
import os
import shutil
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
PATCHER_DIR = os.path.join(os.path.dirname(HERE), "drivingsdk_b200", "patcher")
SELECTED = ("TestMultiScaleDeformableAttentionPatch or TestDeformConvPatch or "
            "TestModulatedDeformConvPatch or TestPatcherIntegration")


def _reference_root():
    root = os.environ.get("MSDA_REFERENCE_ROOT", "")
    test_file = os.path.join(root, "tests", "patcher", "test_patcher_mmcv.py")
    return root if root and os.path.exists(test_file) else None


@pytest.mark.skipif(_reference_root() is None,
                    reason="MSDA_REFERENCE_ROOT does not name a checkout of the reference")
def test_reference_mmcv_hook_tests_pass_on_this_patcher(tmp_path):
    root = _reference_root()
    dst = tmp_path / "mx_driving" / "patcher"
    dst.mkdir(parents=True)
    for name in os.listdir(PATCHER_DIR):
        if name.endswith(".py") and name not in ("__init__.py", "mmcv_patch.py"):
            shutil.copy(os.path.join(PATCHER_DIR, name), dst / name)
    shutil.copy(os.path.join(PATCHER_DIR, "mmcv_patch.py"), dst / "_mmcv_patch_impl.py")
    (dst / "mmcv_patch.py").write_text(
        "import importlib.util, os, sys\n"
        "_spec = importlib.util.spec_from_file_location(\n"
        "    'mx_driving.patcher._mmcv_patch_impl',\n"
        "    os.path.join(os.path.dirname(__file__), '_mmcv_patch_impl.py'))\n"
        "_impl = importlib.util.module_from_spec(_spec)\n"
        "sys.modules[_spec.name] = _impl\n"
        "_spec.loader.exec_module(_impl)\n"
        "globals().update({k: v for k, v in vars(_impl).items() if not k.startswith('__')})\n"
        "SparseConv3D = Stream = DDP = None   # not part of this package\n")
    tests_dir = tmp_path / "tests" / "patcher"
    tests_dir.mkdir(parents=True)
    shutil.copy(os.path.join(root, "tests", "patcher", "test_patcher_mmcv.py"), tests_dir)
    env = dict(os.environ)
    env.pop("PYTHONPATH", None)     # the temporary tree must be the only mx_driving in sight
    proc = subprocess.run(
        [sys.executable, "-m", "pytest", "-q", "-p", "no:cacheprovider",
         str(tests_dir / "test_patcher_mmcv.py"), "-k", SELECTED],
        cwd=str(tmp_path), env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
        timeout=300)
    assert proc.returncode == 0, proc.stdout[-4000:]
    assert " passed" in proc.stdout and "failed" not in proc.stdout, proc.stdout[-2000:]
