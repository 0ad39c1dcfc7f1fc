"""The C-ABI library loads without a GPU and exports every symbol the header
declares; the ABI structs have the reference's layout."""
import ctypes as C
import os
import re

import sme_gemm_b200 as sg
from sme_gemm_b200._lib import SIGNATURES, EpDesc16, EpNode

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "smeg_api.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b(?:int|void|size_t|unsigned|const char \*)\s*\*?\s*((?:smeg|gemm_sme|neon)_\w+)\s*\(", text)
    return sorted(set(names))


def test_library_loads_and_exports_every_declared_symbol():
    lib = sg.lib()
    names = _declared_functions()
    assert len(names) >= 50
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/smeg_api.h but not exported"
    # and the Python binding table covers the same list
    assert sorted(SIGNATURES) == names


def test_epnode_layout_matches_the_reference_struct():
    """csrc/epilogue.h:222-229: 32 bytes, offsets 0/4/8/16/24."""
    assert C.sizeof(EpNode) == 32
    assert [getattr(EpNode, f).offset for f in ("op", "aux", "scalar", "ptr", "ld")] == [0, 4, 8, 16, 24]
    assert C.sizeof(EpDesc16) == 16 and EpDesc16.nodes.offset == 8


def test_version_string():
    assert b"sm_100a" in sg.lib().smeg_version()


def test_bad_arguments_are_rejected_before_any_device_work():
    lib = sg.lib()
    h = C.c_void_p()
    assert lib.smeg_q4_create(None, None, None, 4, 4, 24, C.byref(h)) == -1       # block not a power of two
    assert lib.smeg_q2_create(None, None, 4, 4, 8, (C.c_int8 * 4)(-1, 0, 1, 0), C.byref(h)) == -1   # q2 block < 16
    assert lib.smeg_q1_create(None, None, 0, 4, 4, 1 << 17, C.byref(h)) == -1
    assert lib.smeg_host_pack(3, None, 0, None, 1, 1, 32, None, None) == -4
