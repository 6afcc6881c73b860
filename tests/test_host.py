"""CPU: packer, generator, library loading, argument checking (no GPU needed)."""
import os
import re

import numpy as np
import pytest

import int4linear_b200 as L
from int4linear_b200 import _lib
from conftest import ROOT, golden_files
from oracle import oracle as O


@pytest.mark.parametrize("path", golden_files(), ids=lambda p: p.split("/")[-1][:-4])
def test_packer_matches_golden(path):
    g = np.load(path)
    x = g["x"].astype(np.int32)
    assert np.array_equal(L.pack(x), g["x_packed"])
    assert np.array_equal(L.unpack(g["x_packed"], x.shape[1]), x)
    if x.shape[1] % 8 == 0:
        as_bytes = g["x_packed"].view(np.uint8).reshape(x.shape[0], -1)
        assert np.array_equal(L.pack_bytes(g["x"]), as_bytes)
        assert np.array_equal(L.unpack_bytes(as_bytes), g["x"])


@pytest.mark.parametrize("path", golden_files(), ids=lambda p: p.split("/")[-1][:-4])
def test_native_host_packer_matches_golden(path):
    """The library's own `pack` / `unpack` (C++ symbols with the reference's signatures, and their
    C-ABI aliases) against fixtures produced by the reference's packer."""
    import ctypes
    lib = _lib.load()
    g = np.load(path)
    x = np.ascontiguousarray(g["x"].astype(np.int32))
    m, n = x.shape
    want = np.ascontiguousarray(g["x_packed"]).view(np.int32).reshape(m, -1)
    for pack_name, unpack_name in (("int4_linear_pack_host", "int4_linear_unpack_host"), ("_Z4packPKiPiii", "_Z6unpackPKiPiii")):
        pack_fn, unpack_fn = getattr(lib, pack_name), getattr(lib, unpack_name)
        for fn in (pack_fn, unpack_fn):
            fn.restype, fn.argtypes = None, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
        packed = np.full_like(want, -1)
        pack_fn(x.ctypes.data, packed.ctypes.data, m, n)
        assert np.array_equal(packed, want)
        back = np.empty_like(x)
        unpack_fn(packed.ctypes.data, back.ctypes.data, m, n)
        assert np.array_equal(back, x)


def test_pack_roundtrip_all_values():
    v = np.arange(-8, 8, dtype=np.int32).reshape(1, 16)
    p = L.pack(v)
    assert p.view(np.uint8).ravel()[0] == 0x98  # -8 in the low nibble, -7 in the high one
    assert np.array_equal(L.unpack(p, 16), v)
    assert np.array_equal(O.unpack(p, 16), v)


def test_generator_is_counter_based_and_uniform():
    a = L.uniform_s4(42, 64, 256)
    assert a.min() == -8 and a.max() == 7
    # any row range reproduces the same values
    b = L.uniform_s4(42, 16, 256, row_start=20)
    assert np.array_equal(a[20:36], b)
    p = L.uniform_s4_packed(42, 64, 256, chunk_rows=7)
    assert np.array_equal(p, L.pack_bytes(a))
    ps = L.uniform_s4_packed(42, 8, 256, row_start=40)
    assert np.array_equal(ps, p[40:48])
    counts = np.bincount((L.uniform_s4(1, 512, 512) + 8).ravel(), minlength=16)
    assert counts.min() > 0.9 * counts.mean() and counts.max() < 1.1 * counts.mean()
    assert not np.array_equal(L.uniform_s4(1, 4, 64), L.uniform_s4(2, 4, 64))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "int4linear_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(int4_linear_\w+)\s*\(", header))
    assert declared, "no declarations found in the header"
    lib = _lib.load()
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert declared == set(_lib.SYMBOLS), "ctypes table and header disagree"
    assert lib.int4_linear_version() >= 100


def test_library_exports_the_reference_launcher_symbol():
    """kernels/linear_v21.h:760 of the reference declares `void linear_v21_launch(void*, void*,
    void*, int, int, int)` with C++ linkage; the library exports that mangled symbol and the
    compat directory has the header that declares it."""
    lib = _lib.load()
    name = "linear_v21_launch"
    assert hasattr(lib, f"_Z{len(name)}{name}PvS_S_iii"), name
    hdr = os.path.join(ROOT, "int4linear_b200", "compat", "kernels", "linear_v21.h")
    assert name in open(hdr).read()


def test_argument_checks_need_no_gpu():
    lib = _lib.load()
    buf = np.zeros(4096, dtype=np.uint8)
    base = buf.ctypes.data
    base += (-base) % 16
    ok = (base, base, base)
    assert lib.int4_linear_launch_async(None, base, base, 8, 8, 32, None) == 1
    assert lib.int4_linear_launch_async(*ok, 0, 8, 32, None) == 1
    assert lib.int4_linear_launch_async(*ok, 8, 8, 48, None) == 2      # k % 32 != 0
    assert lib.int4_linear_launch_async(*ok, 8, 8, 131072, None) == 2  # k too large
    assert lib.int4_linear_launch_async(base + 4, base, base, 8, 8, 32, None) == 3
    assert lib.int4_linear_status_string(2).decode().startswith("unsupported")
    assert lib.int4_linear_set_tuning(100, 0, -1) == 1
    assert lib.int4_linear_set_tuning(0, 0, 2) == 1
    assert lib.int4_linear_set_tuning(0, 0, -1) == 0


def test_gather_entry_point_argument_checks_need_no_gpu():
    import ctypes
    lib = _lib.load()
    base = 1 << 20
    ptrs = (ctypes.c_void_p * 2)(base, base + 4096)
    ok = (base, base, None, ptrs)
    assert lib.int4_linear_launch_gather_async(base, base, None, None, 2, 0, 8, 32, 64, 32, None) == 1   # no destinations
    assert lib.int4_linear_launch_gather_async(*ok, 9, 0, 8, 32, 64, 32, None) == 1                      # world > 8
    assert lib.int4_linear_launch_gather_async(*ok, 2, -32, 8, 32, 64, 32, None) == 1                    # negative offset
    bad = (ctypes.c_void_p * 2)(base, base + 4)
    assert lib.int4_linear_launch_gather_async(base, base, None, bad, 2, 0, 8, 32, 64, 32, None) == 1    # misaligned destination
    assert lib.int4_linear_launch_gather_async(*ok, 2, 0, 8, 32, 64, 48, None) == 2                      # k % 32 != 0
    import torch
    from int4linear_b200.linear import linear_gather
    x = torch.zeros((8, 16), dtype=torch.uint8)
    with pytest.raises(ValueError):
        linear_gather(x, x, [base], 0, 8)   # CPU tensors: there is no CPU implementation


def test_no_gpu_means_error_not_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    x = np.zeros((8, 16), dtype=np.uint8)
    with pytest.raises(L.Int4LinearError) as e:
        L.linear_host(x, x, 32)
    assert e.value.status == 6


def test_tile_schedule_covers_every_tile_once(tmp_path):
    """The schedule of the persistent GEMM kernels (whole tiles, half-width items, tiles cut along
    K) is plain host/device arithmetic: tests/schedule_check.cpp enumerates it for tens of thousands
    of (tiles, K blocks, workers) combinations with the host compiler."""
    import subprocess
    exe = str(tmp_path / "schedule_check")
    subprocess.run(["g++", "-O2", "-std=c++17", "-o", exe, os.path.join(ROOT, "tests", "schedule_check.cpp")], check=True)
    out = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and "SCHEDULE_OK" in out.stdout, out.stdout + out.stderr


def test_numa_binding_reads_sysfs_and_keeps_to_allowed_cpus(tmp_path):
    from int4linear_b200 import numa
    assert numa.parse_cpulist("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    dev = tmp_path / "bus" / "pci" / "devices" / "0000:1b:00.0"
    dev.mkdir(parents=True)
    (dev / "numa_node").write_text("1\n")
    node = tmp_path / "devices" / "system" / "node" / "node1"
    node.mkdir(parents=True)
    (node / "cpulist").write_text("48-95\n")
    got = []
    r = numa.bind_to_gpu_node("0000:1B:00.0", sysfs=str(tmp_path), setaffinity=got.append, allowed=set(range(40, 60)))
    assert r == {"node": 1, "cpus": 12, "bound": True} and got == [set(range(48, 60))]
    # no NUMA information (containers often report -1), an unknown device, no usable CPU: nothing is changed
    (dev / "numa_node").write_text("-1\n")
    got.clear()
    assert numa.bind_to_gpu_node("0000:1b:00.0", sysfs=str(tmp_path), setaffinity=got.append)["bound"] is False
    assert numa.bind_to_gpu_node("0000:ff:00.0", sysfs=str(tmp_path), setaffinity=got.append)["bound"] is False
    (dev / "numa_node").write_text("1\n")
    assert numa.bind_to_gpu_node("0000:1b:00.0", sysfs=str(tmp_path), setaffinity=got.append, allowed={1, 2})["bound"] is False
    assert got == []
