"""The C-ABI library loads on a machine without a GPU and exports every symbol that
``include/jetfire_b200.h`` declares; argument errors are reported without a launch."""
import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def lib():
    from jetfire_b200.build import build
    build()
    from jetfire_b200 import _lib
    return _lib


def test_header_symbols_exported(lib):
    header = (ROOT / "include" / "jetfire_b200.h").read_text()
    declared = set(re.findall(r"\b(jf_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations parsed"
    raw = C.CDLL(str(lib.LIB_PATH))
    missing = [n for n in sorted(declared) if not hasattr(raw, n)]
    assert not missing, f"declared but not exported: {missing}"
    assert declared == set(lib.EXPORTED), (declared ^ set(lib.EXPORTED))


def test_status_strings(lib):
    assert lib.status_string(0) == "ok"
    for st in (-1, -2, -3, 1, 2, 3):
        assert lib.status_string(st) not in ("ok", "unknown status")


def test_argument_errors_without_gpu(lib):
    l = lib.lib
    assert l.jf_decode_scan(None, None) == lib.JF_ERR_ARG
    a = lib.DecodeArgs()
    assert l.jf_decode_fused(C.byref(a), None) in (lib.JF_ERR_ARG, lib.JF_ERR_UNSUPPORTED)
    assert l.jf_pack_append(None, 0, 1, 1, 128, 128, None, None, None, 16, 3, 64, None) == lib.JF_ERR_ARG
    assert l.jf_merge_correct(None, None, None, None, None, 0, 1, 1, None) == lib.JF_ERR_ARG
    assert l.jf_decode_workspace_bytes(0, 0, 8, 2, 128, 32) == 0
    assert l.jf_decode_workspace_bytes(0, 1, 32, 8, 32768, 256) > 32 * 32768 * 4


def test_struct_layout_matches_header(lib):
    # twelve 4-byte fields, one int64, sixteen pointers, one uint64, one more pointer
    assert C.sizeof(lib.DecodeArgs) == 48 + 8 + 16 * 8 + 8 + 8
    assert lib.DecodeArgs.num_slots.offset == 48
    assert lib.DecodeArgs.q.offset == 56
    assert lib.DecodeArgs.workspace_bytes.offset == 56 + 16 * 8
    assert lib.DecodeArgs.topk_slots_i32.offset == 56 + 16 * 8 + 8


def test_status_of_a_host_copy_of_the_record(lib):
    """The non-synchronising status check reads a 16-byte host copy of the workspace's record:
    only a tagged record with a non-zero code counts."""
    import struct
    l = lib.lib
    tag = struct.unpack("<Q", b"SUTATSFJ")[0]           # "JFSTATUS" as the kernels write it
    assert tag == 0x4A46535441545553
    rec = lambda t, code: C.create_string_buffer(struct.pack("<Qii", t, code, 0), 16)
    assert l.jf_decode_status_of_copy(rec(tag, 0)) == lib.JF_OK
    assert l.jf_decode_status_of_copy(rec(tag, 2)) == lib.JF_ERR_TIMEOUT
    assert l.jf_decode_status_of_copy(rec(tag, 3)) == lib.JF_ERR_STATE
    assert l.jf_decode_status_of_copy(rec(0x1234, 2)) == lib.JF_OK          # whatever the workspace held before
    assert l.jf_decode_status_of_copy(None) == lib.JF_ERR_ARG
