"""The checked build of the library (adaptq_b200/libadaptq_b200_checked.so: the same
sources compiled with -DADAPTQ_CHECKED) runs the awkward-shape, append, compute and
streaming tests in a child process.  In that build every store and every row read is
preceded by an index check that records a status word instead of trapping, every device
buffer is followed by guard bytes, and adaptq_mha_synchronize() reports a failed check or
a damaged guard -- the stand-in for a memory checker on machines where none may run.
A passing run therefore means: same results, no out-of-range index, no write past a buffer."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CHECKED = os.path.join(ROOT, "adaptq_b200", "libadaptq_b200_checked.so")


def test_suites_pass_under_the_checked_build(gpu_lib):
    if not os.path.exists(CHECKED):
        pytest.skip("libadaptq_b200_checked.so not built (python -m adaptq_b200.build --checked)")
    env = dict(os.environ, ADAPTQ_B200_LIB=CHECKED)
    probe = subprocess.run([sys.executable, "-c", "import adaptq_b200; print(adaptq_b200.load().adaptq_version().decode())"],
                           capture_output=True, text=True, env=env, cwd=ROOT, timeout=300)
    assert probe.stdout.strip().endswith("-sm100a-checked"), probe.stdout + probe.stderr
    files = ["tests/test_gpu_tiny_shapes.py", "tests/test_gpu_append.py", "tests/test_gpu_decode_step.py",
             "tests/test_gpu_stack.py", "tests/test_gpu_compute.py"]
    r = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu", "-p", "no:cacheprovider", *files],
                       capture_output=True, text=True, env=env, cwd=ROOT, timeout=3000)
    assert r.returncode == 0, r.stdout[-6000:] + r.stderr[-2000:]
