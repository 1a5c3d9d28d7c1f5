"""The C-ABI library loads on a CPU-only machine and exports every symbol the header declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "pce_b200.h")).read()
    return sorted(set(re.findall(r"PCE_API[^;(]*?\b(pce_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    import __graft_entry__ as ge
    ge.build()
    lib = ctypes.CDLL(os.path.join(ROOT, "pcengine_b200", "libpce_b200.so"))
    names = _declared()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), n
    from pcengine_b200 import _lib
    assert sorted(_lib.EXPORTS) == names


def test_status_strings_and_size_queries_need_no_gpu():
    from pcengine_b200._lib import lib
    assert lib.pce_strerror(0) == b"ok"
    assert b"workspace" in lib.pce_strerror(3)
    assert lib.pce_version() >= 100
    assert lib.pce_map_workspace_bytes(100000, 27, 100000) > 16 * 262144
    assert lib.pce_csr_from_pairs_workspace_bytes(1000, 100) > 0


def test_product_refuses_cpu_tensors():
    import pytest
    import torch

    import pcengine_b200 as pce
    coords = torch.zeros((4, 4), dtype=torch.int32)
    with pytest.raises(RuntimeError):
        pce.KernelMap(coords, (3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0], [1, 1, 1], True)
    with pytest.raises(RuntimeError):
        pce.functional.linear_forward(torch.zeros(4, 4), torch.zeros(4, 4))


def test_package_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "pcengine_b200")
    for base, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(base, f)).read()
                assert "oracle" not in src, os.path.join(base, f)


def test_ctypes_mirrors_match_the_header_layout(tmp_path):
    """The header compiled as plain C: size of every struct and offset of its last field equal the
    ctypes mirrors' (a field added on one side only would shift everything behind it)."""
    import subprocess

    from pcengine_b200 import _lib
    pairs = [("pce_geom", _lib.Geom), ("pce_tile_lists", _lib.TileLists), ("pce_epilogue", _lib.Epilogue),
             ("pce_plan_map_spec", _lib.PlanMapSpec), ("pce_planned_csr", _lib.PlannedCSR),
             ("pce_planned_map", _lib.PlannedMap)]
    lines = []
    for cname, mirror in pairs:
        last = mirror._fields_[-1][0]
        lines.append(f'printf("{cname} %zu %zu\\n", sizeof({cname}), offsetof({cname}, {last}));')
    src = tmp_path / "layout.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "pce_b200.h"\nint main(void) {\n'
                   + "\n".join(lines) + "\nreturn 0; }\n")
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c99", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split("\n")
    seen = {}
    for line in out:
        if line:
            name, size, off = line.split()
            seen[name] = (int(size), int(off))
    for cname, mirror in pairs:
        last = mirror._fields_[-1][0]
        assert seen[cname] == (ctypes.sizeof(mirror), getattr(mirror, last).offset), cname
