"""Variants of a kernel library built with preprocessor definitions: a file of their own beside the plain
build, with the marks compiled in."""
import ctypes
import os

from sglang_rs_b200.csrc import build


def test_a_timeline_variant_is_a_file_of_its_own_and_exports_its_switch():
    plain = build.compile_library("elementwise")
    variant = build.compile_library("elementwise", ("SRB_TIMELINE",))
    assert plain != variant and os.path.exists(plain) and os.path.exists(variant)
    assert "+SRB_TIMELINE-" in os.path.basename(variant)
    assert build.compile_library("elementwise", ("SRB_TIMELINE",)) == variant          # found again, not rebuilt
    library = ctypes.CDLL(variant)
    assert hasattr(library, "srb_set_timeline")
    assert not hasattr(ctypes.CDLL(plain), "srb_set_timeline")
