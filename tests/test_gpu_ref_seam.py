"""The reference's own SampleBuffers / filterCands / sampleRow / Acceptor, unmodified, running over this library's kernels
through ServerModel::topkRows and Backend::download (oracle/ref_on_gpu.cpp, built where a reference checkout exists).
Every seeded case must give the same accept count, chosen token, kept-set size and escalation counters as the same code
over the reference's host double."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "oracle", "_ref", "ref_on_gpu")


def test_reference_host_code_over_gpu_kernels():
    if not os.path.exists(EXE):
        pytest.skip("oracle/_ref/ref_on_gpu not built (no reference checkout when the tree was prepared)")
    out = subprocess.run([EXE, "80"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "80 / 80 cases identical" in out.stdout and "argmax ok" in out.stdout, out.stdout
