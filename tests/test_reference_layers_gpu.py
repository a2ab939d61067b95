"""The reference's own layer self-checks, run unchanged on this package's operators.

Each layer module of the reference (`flash_bla/layers/*.py`) ends in a self-test that builds the layer on the
GPU and compares its `mode='triton'` path -- which calls `linear_attention` / `decoupled_la` from
`flash_bla.ops` -- with its dense `mode='torch'` path, outputs and input gradients.  Here the layer files of an
installed copy of the reference (`baseline/_ref`, not part of this repository) are copied to a temporary
directory and executed with this package providing `flash_bla.ops` and `flash_bla.utils`.  The LinFusion layer
needs `diffusers`, which this image does not have.
"""
import os
import shutil
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "flash-bidirectional-linear-attention_b200")
REF_LAYERS = os.path.join(ROOT, "baseline", "_ref", "flash_bla", "layers")


@pytest.mark.skipif(not os.path.isdir(REF_LAYERS), reason="no installed copy of the reference under baseline/_ref")
@pytest.mark.parametrize("layer", ["mlla", "rala", "polaformer", "focused_la"])
def test_reference_layer_self_check(layer, tmp_path):
    dst = tmp_path / "flash_bla" / "layers"          # a namespace portion: no __init__.py on purpose
    dst.mkdir(parents=True)
    for name in ("mlla", "rala", "polaformer", "focused_la"):
        shutil.copy(os.path.join(REF_LAYERS, name + ".py"), dst / (name + ".py"))
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([PKG, str(tmp_path)]), FLASH_BLA_PRINT_ERR="1")
    r = subprocess.run([sys.executable, "-m", f"flash_bla.layers.{layer}"], env=env, capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "match" in r.stdout, r.stdout[-2000:]
    # the layers run in fp32: the RMS error ratio their own check tolerates is 6e-2, ours is 1e-3
    import re
    ratios = [float(x) for x in re.findall(r"ratio: ([0-9.eE+-]+)", r.stdout)]
    assert all(x < 1e-3 for x in ratios), r.stdout[-2000:]


REF_VARLEN_TEST = os.path.join(ROOT, "baseline", "_ref", "tests", "ops", "test_varlen_linear_attn.py")


@pytest.mark.skipif(not os.path.exists(REF_VARLEN_TEST), reason="the reference's test file is not staged under baseline/_ref/tests")
def test_reference_varlen_pytest_runs_unchanged(tmp_path):
    """The reference's only pytest file (tests/ops/test_varlen_linear_attn.py: 32 parameter combinations of
    varlen forward + backward against its dense torch statement, and the oversized-max_seqlen case), copied
    as it is to a temporary directory and run in a child process with this package providing ``flash_bla``."""
    shutil.copy(REF_VARLEN_TEST, tmp_path / "test_varlen_linear_attn.py")
    env = dict(os.environ, PYTHONPATH=PKG)
    r = subprocess.run([sys.executable, "-m", "pytest", "-q", "-p", "no:cacheprovider", "--rootdir", str(tmp_path),
                        str(tmp_path / "test_varlen_linear_attn.py")], env=env, capture_output=True, text=True,
                       timeout=900, cwd=str(tmp_path))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert "33 passed" in r.stdout, r.stdout[-1000:]
