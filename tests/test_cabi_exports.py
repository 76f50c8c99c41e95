"""The C-ABI library loads without a GPU and exports every symbol include/neus2b.h declares; host-only entry points
(level table, parameter counts, pcg32) agree with the oracle."""
import os
import re

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from neus2_b200 import _lib as L
    from neus2_b200 import build
    build.build()
    lib = L.lib()
    hdr = open(os.path.join(ROOT, "include", "neus2b.h")).read()
    declared = set(re.findall(r"\b(neus2b_[a-z0-9_]+)\s*\(", hdr))
    assert declared, "header parse"
    for sym in sorted(declared):
        assert hasattr(lib, sym), "missing export " + sym
    assert declared == set(L.EXPORTS), declared ^ set(L.EXPORTS)
    assert b"sm_100a" in lib.neus2b_version()


def test_level_table_and_counts_match_oracle(oracle):
    from neus2_b200 import _lib as L
    for kw in (dict(), dict(n_levels=14, per_level_scale=1.4525), dict(n_levels=4, log2_hashmap_size=10, base_resolution=4, per_level_scale=1.7)):
        d, od = L.grid_desc(**kw), oracle.grid_desc(**kw)
        assert L.grid_n_params(d) == oracle.grid_n_params(od)
        assert L.model_n_params(d) == oracle.model_n_params(od)
        off, res, scale, hashed = L.grid_level_table(d)
        lv = oracle.grid_levels(od)
        nl = d.n_levels
        assert off[:nl + 1] == list(lv.offset)[:nl + 1] and res == list(lv.res) and hashed == list(lv.hashed)
        assert np.array_equal(np.float32(scale), np.float32(list(lv.scale)))
    d = L.grid_desc()
    # BASELINE config 0: 5 dense + 11 hashed levels, ~12.6 M parameters
    assert sum(L.grid_level_table(d)[3]) == 11 and L.grid_n_params(d) == 12599920


def test_bad_arguments_are_rejected_without_a_gpu():
    import ctypes as C
    from neus2_b200 import _lib as L
    bad = L.GridDesc(17, 19, 16, 1.447, 17)
    n = C.c_uint64(0)
    assert L.lib().neus2b_grid_n_params(C.byref(bad), C.byref(n)) == -1
    d = L.grid_desc()
    assert L.lib().neus2b_grid_forward(C.byref(d), 16, None, 3, None, None, None, None) == -1
    assert L.lib().neus2b_mlp_forward(16, 40, 1, C.c_void_p(16), C.c_void_p(16), C.c_void_p(16), None, None) == -2
    assert L.lib().neus2b_error_string(-2) == b"unsupported configuration"


def test_pcg32_host(oracle):
    from neus2_b200 import _lib as L
    a, b = L.pcg32(1337), oracle.pcg32(1337)
    assert (a.state, a.inc) == (b.state, b.inc)
    a, b = L.pcg32_advance(a, 2 ** 40 + 5), oracle.pcg32_advance(b, 2 ** 40 + 5)
    assert a.state == b.state
