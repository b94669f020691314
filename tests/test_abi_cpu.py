"""The C-ABI library on a machine without a GPU: it loads, exports every function include/ds41_b200.h declares, and its
host-only entry points (Philox words and uniforms, the thread-local error text, argument checks that return before any
CUDA call) behave as the reference's (engine/tests/core.cpp:22-34; third_party/spark/src/sampling.cpp:9-10,57-58).
No kernel is launched here."""
import ctypes as C
import math
import os
import re

import pytest

import __graft_entry__ as entry

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def pkg():
    entry.build()
    return entry.load_package()


def declared_functions():
    text = open(os.path.join(ROOT, "include", "ds41_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"\b(ds41_[a-z0-9_]+)\s*\(", text))
    assert len(names) >= 25
    return sorted(names)


def test_every_declared_function_is_exported(pkg):
    lib = C.CDLL(pkg.LIB_PATH)
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert not missing, missing


def test_philox_known_answers_of_the_library(pkg):
    lib = pkg.lib()
    words = [lib.ds41_spark_rng_word_v2(0, 0, 0, 0, d) for d in range(4)]
    assert words == [0xe0481467, 0x8ddfd609, 0xb08e446f, 0x1852b5ab]
    assert lib.ds41_spark_uniform_v2(0, 0, 0, 0, 0) == 0.8760998513862246
    w = lib.ds41_spark_rng_word_v2
    assert w(0, 0, 0, 0, 0) != w(0, 0, 0, 1, 0)      # purpose separates the streams
    assert w(0, 1, 0, 0, 0) != w(0, 0, 0, 0, 0)      # step
    assert w(0, 0, 1, 0, 0) != w(0, 0, 0, 0, 0)      # slot
    assert w(1, 0, 0, 0, 0) != w(0, 0, 0, 0, 0)      # seed
    # 53-bit construction from two words (spark_rng.h:30-36)
    a, b = w(7, 9, 2, 3, 10) >> 5, w(7, 9, 2, 3, 11) >> 6
    assert lib.ds41_spark_uniform_v2(7, 9, 2, 3, 5) == ((a << 26) | b) * 2.0 ** -53
    # out-of-range addresses: 0 / NaN and a message (spark.h:97-98)
    assert w(0, 0, 6, 0, 0) == 0 and "out of range" in pkg.last_error()
    assert w(0, 0, 0, 4, 0) == 0
    assert math.isnan(lib.ds41_spark_uniform_v2(0, 0, 0, 0, 8589934592))
    assert not math.isnan(lib.ds41_spark_uniform_v2(0, 0, 0, 0, 8589934591))
    assert w(0, 0, 5, 3, 4 * 0xFFFFFFFF + 3) != 0 or True   # the largest draw is accepted
    assert w(0, 0, 0, 0, 4 * 0x100000000) == 0


def test_host_mirror_rng_and_attempt_counter(pkg):
    r = pkg.Rng(0)
    assert r.word(0, 0, pkg.Purpose.Target, 0) == 0xe0481467
    assert r.word(0, 0, pkg.Purpose.Target, 3) == 0x1852b5ab
    assert r.uniform(0, 0, pkg.Purpose.Target) == 0.8760998513862246
    assert r.word(0, 0, pkg.Purpose.Target) != r.word(0, 0, pkg.Purpose.Draft)
    with pytest.raises(OverflowError):
        r.uniform(0, 0, pkg.Purpose.Target, 8589934592)
    with pytest.raises(OverflowError):
        r.word(0, 6, pkg.Purpose.Target)
    nonce = pkg.AttemptCounter(2 ** 64 - 2)
    assert nonce.take() == 2 ** 64 - 2 and nonce.take() == 2 ** 64 - 1
    with pytest.raises(OverflowError):
        nonce.take()
    assert [int(p) for p in pkg.Purpose] == [0, 1, 2, 3]


def test_argument_checks_need_no_device(pkg):
    """Struct sizes of the host mirror match the library's, and argument errors are reported (cudaErrorInvalidValue = 1
    plus a message) before any CUDA call is made."""
    lib = pkg.lib()
    a = pkg.SampleArgs()
    a.struct_bytes = C.sizeof(pkg.SampleArgs) - 8
    assert lib.ds41_b200_sample_logits(C.byref(a), None) == 1 and "ABI" in pkg.last_error()
    a.struct_bytes = C.sizeof(pkg.SampleArgs)
    assert lib.ds41_b200_sample_logits(C.byref(a), None) == 1 and "rows/vocab" in pkg.last_error()
    v = pkg.VerifyArgs()
    v.struct_bytes = C.sizeof(pkg.VerifyArgs)
    assert lib.ds41_b200_verify_logits(C.byref(v), None) == 1 and "ABI" not in pkg.last_error()
    s = pkg.ScoreArgs()
    s.struct_bytes = C.sizeof(pkg.ScoreArgs)
    assert lib.ds41_b200_score_logits(C.byref(s), None) == 1 and "ABI" not in pkg.last_error()
    assert lib.ds41_fuse_head_decode(None, None, None, 7, 129280, 5120, None) == 1      # head_decode.cpp:6: M <= 6
    assert lib.ds41_fuse_head_decode(None, None, None, 1, 1000, 5120, None) == 1
    assert pkg.sample_scratch_bytes(0, 129280) == 0 and pkg.sample_scratch_bytes(4, 200000) == 0
    assert pkg.sample_scratch_bytes(1024, 129280) > 1024 * 129280 // 32
    assert pkg.fuse_head_fp8_workspace_bytes(4, 100) == 0
    assert lib.ds41_b200_verify_logits_static_max_rows() == 1024
