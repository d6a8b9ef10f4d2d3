"""The call half of the drop-in check (needs a B200): tests/abi/contract.c, compiled against the REFERENCE's
src/gpu.h and src/weights/residency.h only and linked with libh3q8.so, creates a context, runs a bf16 linear
through the reference's prototypes and reads the counters back through the reference's h3_gpu_stats."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
BINARY = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "abi_contract")


def test_reference_header_client_runs_on_the_library():
    if not os.path.exists(BINARY):
        pytest.skip("oracle/_ref/abi_contract was not built (no reference tree at build time)")
    result = subprocess.run([BINARY, "run"], capture_output=True, text=True, timeout=120)
    assert result.returncode == 0, result.stderr
    assert "contract run ok" in result.stdout
