"""The C ABI: the shared library loads, exports exactly what include/slora_b200.h declares, and rejects bad
arguments with status codes before touching the device (no GPU needed)."""
import ctypes
import os
import re

from tests.helpers import ROOT
from slora_b200 import _lib


def _header_functions():
    text = open(os.path.join(ROOT, "include", "slora_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    out = {}
    for m in re.finditer(r"\b(?:int|void|size_t|const char\*)\s+(slora_\w+)\s*\(([^;]*?)\)\s*;", text, flags=re.S):
        args = m.group(2).strip()
        out[m.group(1)] = 0 if args == "void" else len(args.split(","))
    return out


def test_library_exports_every_declared_symbol_and_nothing_else():
    declared = _header_functions()
    assert set(declared) == set(_lib.EXPORTS)
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared:
        assert getattr(lib, name) is not None


def test_binding_argument_counts_match_header():
    declared = _header_functions()
    for name, (_, args) in _lib._SIGS.items():
        assert len(args) == declared[name], name


def test_version_and_workspace_size():
    assert _lib.lib.slora_version() >= 100
    small = _lib.lib.slora_plan_workspace_bytes(256, 1000)
    big = _lib.lib.slora_plan_workspace_bytes(4096, 2000)
    assert 0 < small < big
    # header + tiles + perm + pos + counters
    assert small >= 4 * (16 + 8 * (32 + 256) + 2 * 256 + 1000)
    assert _lib.lib.slora_plan_workspace_bytes(-1, 5) == 0
    # resolved tiles: 12 + 4 * cap words per tile slot on top, cap = max_rank rounded up to a multiple of 8
    assert _lib.lib.slora_plan_workspace_bytes_ex(256, 1000, 0) == small
    with_tiles = _lib.lib.slora_plan_workspace_bytes_ex(256, 1000, 12)
    assert with_tiles >= small + 4 * (32 + 256) * (12 + 4 * 16) and with_tiles - small < 4 * (32 + 256) * (12 + 4 * 16) + 64
    assert _lib.lib.slora_plan_workspace_bytes_ex(256, 1000, 129) == small      # beyond the cap: none
    assert _lib.flag_resolved(12) == 2 << 8 and _lib.flag_resolved(0) == 0 and _lib.flag_resolved(128) == 16 << 8


def test_argument_validation_needs_no_device():
    L = _lib.lib
    fake = 0x1000  # 16-byte aligned, never dereferenced: validation fails first
    # null pool
    rc = L.slora_bgmv_shrink(fake, fake, 0, fake, fake, fake, fake, 0, 4, 1024, 1024, 8, 8, 64, 1024, 2, 64, 0, 0)
    assert rc == -1 and "null" in _lib.last_error()
    # dtype
    rc = L.slora_bgmv_shrink(fake, fake, fake, fake, fake, fake, fake, 0, 4, 1024, 1024, 8, 8, 64, 1024, 2, 64, 7, 0)
    assert rc == -3
    # h_in not a multiple of 8
    rc = L.slora_bgmv_shrink(fake, fake, fake, fake, fake, fake, fake, 0, 4, 1020, 1020, 8, 8, 64, 1024, 2, 64, 0, 0)
    assert rc == -4 and "No suitable kernel" in _lib.last_error()
    # misaligned activations
    rc = L.slora_bgmv_shrink(fake, fake + 2, fake, fake, fake, fake, fake, 0, 4, 1024, 1024, 8, 8, 64, 1024, 2, 64, 0, 0)
    assert rc == -2
    # projection index
    rc = L.slora_bgmv_shrink(fake, fake, fake, fake, fake, fake, fake, 5, 4, 1024, 1024, 8, 8, 64, 1024, 2, 64, 0, 0)
    assert rc == -5
    # rank beyond the expand path
    rc = L.slora_bgmv_expand(fake, fake, fake, fake, fake, fake, fake, fake, 0, 4, 1024, 256, 256, 1024, 64, 1024, 2,
                             64, 0, 0)
    assert rc == -8
    # plan workspace too small
    rc = L.slora_plan_build(fake, 16, fake, 256, fake, fake, 1000, 64, 0)
    assert rc == -6
    # an empty batch is a no-op, not an error
    rc = L.slora_bgmv_shrink(fake, fake, fake, fake, fake, fake, fake, 0, 0, 1024, 1024, 8, 8, 64, 1024, 2, 64, 0, 0)
    assert rc == 0
