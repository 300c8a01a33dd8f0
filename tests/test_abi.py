"""CPU tests of the boundary: the shared library loads, exports every function that
include/b200attn.h declares, validates arguments without touching a device, and its shard-range
helper partitions (batch, head) slices exactly."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "b200attn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\([^;{]*\)\s*;", text)))


def test_header_declares_the_drop_in_symbols(pkg):
    names = declared_functions()
    for s in pkg.DROP_IN_SYMBOLS:
        assert s in names
    assert "b200attn_forward_ex" in names and "b200attn_forward_sharded" in names


def test_library_exports_every_declared_symbol(pkg):
    L = pkg.lib()
    for name in declared_functions():
        assert hasattr(L, name), f"{name} declared in include/b200attn.h but not exported"


def test_args_struct_matches_header(pkg):
    # 4 pointers + 5 ints + 3 ints + float + 2 pointers + pointer + unsigned, natural alignment
    assert C.sizeof(pkg.Args) == 8 + 4 * 8 + 5 * 4 + 3 * 4 + 4 + 4 + 2 * 8 + 8 + 8
    assert pkg.Args.stream.offset % 8 == 0


def test_validation_needs_no_device(pkg):
    L = pkg.lib()
    assert L.b200attn_forward_ex(None) == 1
    assert b"NULL" in L.b200attn_last_error()
    a = pkg.make_args(0, 0, 0, 0, 1, 1, 4, 4, 8, pkg.F32)
    assert L.b200attn_forward_ex(C.byref(a)) == 1
    a = pkg.make_args(16, 32, 48, 64, 1, 1, 0, 4, 8, pkg.F32)
    assert L.b200attn_forward_ex(C.byref(a)) == 1 and b"positive" in L.b200attn_last_error()
    a = pkg.make_args(16, 32, 48, 64, 1, 1, 4, 4, 8, 7)
    assert L.b200attn_forward_ex(C.byref(a)) == 1
    a = pkg.make_args(16, 32, 48, 64, 1, 1, 4, 4, 8, pkg.F32, pe=pkg.PE_ROPE_HALF, rotary_dim=6 + 1)
    assert L.b200attn_forward_ex(C.byref(a)) == 1 and b"rotary_dim" in L.b200attn_last_error()
    a = pkg.make_args(16, 32, 48, 16, 1, 1, 4, 4, 8, pkg.F32)
    assert L.b200attn_forward_ex(C.byref(a)) == 1 and b"alias" in L.b200attn_last_error()
    a = pkg.make_args(18, 32, 48, 64, 1, 1, 4, 4, 8, pkg.F32)
    assert L.b200attn_forward_ex(C.byref(a)) == 1 and b"aligned" in L.b200attn_last_error()
    bad = pkg.make_args(16, 32, 48, 64, 1, 1, 4, 4, 8, pkg.F32)
    bad.struct_size = 8
    assert L.b200attn_forward_ex(C.byref(bad)) == 1 and b"struct_size" in L.b200attn_last_error()


@pytest.mark.parametrize("total,n", [(512, 8), (128, 4), (4, 8), (7, 3), (1, 1), (0, 2)])
def test_shard_ranges_partition(pkg, total, n):
    begin, count = pkg.shard_ranges(total, n)
    assert sum(count) == total and begin[0] == 0
    for g in range(1, n):
        assert begin[g] == begin[g - 1] + count[g - 1]
    assert max(count) - min(count) <= 1


def test_version_and_counters(pkg):
    assert b"b200attn" in pkg.lib().b200attn_version()
    assert pkg.launch_count() >= 0
