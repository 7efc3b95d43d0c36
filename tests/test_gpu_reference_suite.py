"""The reference project's own operator test-suite, unmodified, against this package.

The reference ships ``python -m tests --part ops`` (unittest; tests/__main__.py:104-161 of the reference), which
imports only ``ramnet_ops`` and ``torch.ops.ramnet_ops.*``: schema / fake-tensor / autograd registration checks
(torch.library.opcheck), torch.compile (aot_eager and inductor, full graph, no recompiles, CUDA-graph replay),
behaviour (chunked == full, in place == functional, masks) and numerics against its PyTorch backend, in fp32 and,
with --bf16 --fp16, in the 16-bit types.  This test runs that suite in a subprocess with this package first on the
import path.  It needs a checkout of the reference, which is not part of this repository: set the environment
variable RAMNET_REFERENCE_ROOT to a directory that holds the reference's ``tests`` package; without it the test is
skipped.  RAMNET_REFERENCE_SUITE_LOG names a file that receives the suite's full output.
tests/reference_suite_result.md holds the result of the last run on a B200.
"""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent


def test_reference_operator_suite_passes_unmodified():
    ref_root = os.environ.get("RAMNET_REFERENCE_ROOT", "")
    if not ref_root or not (Path(ref_root) / "tests" / "__main__.py").exists():
        pytest.skip("RAMNET_REFERENCE_ROOT does not point at a checkout of the reference (with its tests package)")
    env = dict(os.environ)
    env["PYTHONPATH"] = str(ROOT / "ram-net_b200") + os.pathsep + env.get("PYTHONPATH", "")
    env["PYTHONDONTWRITEBYTECODE"] = "1"
    seeds = os.environ.get("RAMNET_REFERENCE_SEEDS", "0 1 2").split()
    res = subprocess.run([sys.executable, "-m", "tests", "--part", "ops", "--device", "cuda", "--bf16", "--fp16", "--seeds", *seeds],
                         cwd=ref_root, env=env, capture_output=True, text=True, timeout=3000)
    log = res.stdout + res.stderr
    log_path = os.environ.get("RAMNET_REFERENCE_SUITE_LOG", "")
    if log_path:
        Path(log_path).write_text(log)
    assert "ram-net_b200" in log, "the suite must have imported this package, not the reference's"
    assert res.returncode == 0, "reference suite failed:\n" + log[-4000:]
