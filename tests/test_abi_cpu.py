"""The C-ABI library loads without a GPU and exports every function include/*.h declares;
argument validation that needs no device work is exercised too."""
import ctypes as C
import glob
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    names = set()
    for path in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = re.sub(r"/\*.*?\*/", "", open(path).read(), flags=re.S)
        names.update(re.findall(r"\b(ri_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol():
    from retrievalattention_b200 import _lib

    names = declared_functions()
    assert "ri_wave_decode_layer" in names and len(names) >= 8
    missing = [n for n in names if not hasattr(_lib.lib, n)]
    assert not missing, f"declared in include/ but not exported: {missing}"
    assert _lib.lib.ri_version() >= 1


def test_struct_mirror_matches_header_field_order():
    from retrievalattention_b200 import _lib

    text = open(os.path.join(ROOT, "include", "ri_b200.h")).read()
    body = text[text.index("typedef struct ri_wave_layer {"):text.index("} ri_wave_layer;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = re.findall(r"\b([a-z_0-9]+)\s*;", body)
    assert fields == [f[0] for f in _lib.WaveLayer._fields_]


def test_geometry_is_validated_without_a_device():
    from retrievalattention_b200 import _lib

    p = _lib.WaveLayer()
    assert _lib.lib.ri_wave_scratch_bytes(C.byref(p)) == -1
    p.groups, p.group_size, p.n_centroids, p.nprobe, p.n_estimate = 4, 9, 64, 4, 8
    p.page_size, p.buffer_pages, p.steady_stride, p.max_exact_rows = 8, 16, 76, 128
    assert _lib.lib.ri_wave_scratch_bytes(C.byref(p)) == -1
    assert b"group_size" in _lib.lib.ri_last_error()
    p.group_size = 4
    assert _lib.lib.ri_wave_scratch_bytes(C.byref(p)) > 0
    p.n_centroids = 60
    assert _lib.lib.ri_wave_scratch_bytes(C.byref(p)) == -1


def test_config_derivation_matches_reference_table():
    """benchmark/config.py:34-53 for the five benchmark configurations."""
    from retrievalattention_b200.config import GEOMETRIES

    expect = {"cfg0": (512, 1, 9, 127), "cfg1": (8192, 16, 147, 2047), "cfg3": (16384, 32, 294, 4095),
              "cfg4": (8192, 16, 147, 2047)}
    for name, (c, seg, p, mc) in expect.items():
        cfg = GEOMETRIES[name].index()
        assert (cfg.n_centroids, cfg.n_segment, cfg.nprobe, cfg.max_compute_cluster_num) == (c, seg, p, mc)
        assert cfg.cache_cluster_num == 3 * p
