"""CPU-side checks of the C-ABI library: it loads, exports every symbol the
headers declare, and refuses to work without a GPU (no CPU fallback)."""
import ctypes
import glob
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        src = open(h).read()
        src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
        names |= set(re.findall(r"\b(dpb_[a-z0-9_]+)\s*\(", src))
    return sorted(names)


def test_header_symbols_exported(dpb):
    names = declared_symbols()
    assert len(names) >= 25
    for n in names:
        assert hasattr(dpb.lib, n), f"{n} is declared in include/ but not exported by libdpb.so"


def test_bindings_cover_header(dpb):
    assert set(dpb.SIGNATURES) <= set(declared_symbols())


def test_no_cpu_fallback(dpb):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(dpb.DpbError) as e:
        dpb.Context(0)
    assert e.value.code == dpb.ECUDA
    assert "no CPU path" in str(e.value)


def test_library_does_not_link_the_oracle(dpb):
    # the shipped library must not depend on test infrastructure
    with open(dpb.LIB_PATH, "rb") as f:
        blob = f.read()
    assert b"liboracle" not in blob
