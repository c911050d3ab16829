"""The C-ABI library loads on a machine without a GPU and exports what include/b200q.h declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200q.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200q_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/b200q.h but not exported"


def test_binding_table_matches_header():
    from gomlx_b200 import _native
    assert sorted(_native.SYMBOLS) == declared_symbols()


def test_metadata(lib):
    assert lib.b200q_version() >= 100
    for t, bpb, vpb, name, dec in [(2, 18, 32, b"Q4_0", 1), (8, 34, 32, b"Q8_0", 1), (12, 144, 256, b"Q4_K", 0),
                                   (14, 210, 256, b"Q6_K", 0), (20, 18, 32, b"IQ4_NL", 1)]:
        assert lib.b200q_ggml_bytes_per_block(t) == bpb
        assert lib.b200q_ggml_values_per_block(t) == vpb
        assert lib.b200q_ggml_type_name(t) == name
        assert lib.b200q_ggml_can_decompose(t) == dec
    assert lib.b200q_ggml_bytes_per_block(99) == 0
    assert lib.b200q_ggml_type_name(99) is None


def test_shard_rows_partition(lib):
    from gomlx_b200 import shard_rows
    for n in (16, 100, 1024, 4096, 14336, 28672, 8192, 17):
        for world in (1, 2, 4, 8):
            ranges = [shard_rows(n, r, world) for r in range(world)]
            pos = 0
            for b, c in ranges:
                assert b == pos and c >= 0
                pos += c
            assert pos == n
            assert all(b % 16 == 0 for b, c in ranges if c > 0)
    assert [c for _, c in [shard_rows(28672, r, 8) for r in range(8)]] == [3584] * 8


def test_argument_errors_without_gpu(lib):
    from gomlx_b200 import _native as nat
    h = ctypes.c_uint64()
    data = (ctypes.c_uint8 * 34)()
    # validation happens before any CUDA call
    assert lib.b200q_weight_upload(0, 8, 1, 31, data, 34, 0, ctypes.byref(h)) == nat.EINVAL
    assert b"multiple" in lib.b200q_last_error()
    assert lib.b200q_weight_upload(0, 8, 1, 32, data, 33, 0, ctypes.byref(h)) == nat.EINVAL
    assert lib.b200q_weight_upload(0, 20, 1, 32, data, 18, 0, ctypes.byref(h)) == nat.ENOTIMPL
    assert lib.b200q_weight_upload(0, 3, 1, 32, data, 18, 0, ctypes.byref(h)) == nat.ENOTIMPL
    assert lib.b200q_weight_free(12345) == nat.EHANDLE
    assert lib.b200q_dense(777, None, 0, 1, None, 0, None, 0, None) == nat.EHANDLE
    assert lib.b200q_weight_live_count() == 0
    with pytest.raises(nat.B200QError):
        nat.check(lib.b200q_weight_free(1))
