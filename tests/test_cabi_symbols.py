"""The C-ABI library loads without a GPU, exports every function include/b200fp8.h declares, and
answers the calls that need no device."""
import ctypes
import os
import re

import pytest

from tritonbench_b200 import lib
from tritonbench_b200.csrc import build as csrc_build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "b200fp8.h")


@pytest.fixture(scope="module")
def cdll():
    if not os.path.exists(lib.LIB_PATH):
        csrc_build.build()
    return lib.load()


def _declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200fp8_[a-z_0-9]+)\s*\(", text)))


def test_header_and_binding_list_the_same_functions():
    assert _declared_functions() == sorted(lib.EXPORTED_SYMBOLS)


def test_every_declared_symbol_is_exported(cdll):
    for name in _declared_functions():
        assert hasattr(cdll, name), name


def test_abi_version_and_status_strings(cdll):
    assert cdll.b200fp8_abi_version() == 1
    seen = {lib.status_string(s) for s in range(8)}
    assert len(seen) == 8 and "ok" in seen
    assert lib.status_string(99) == "unknown status"


def test_null_pointers_and_bad_sizes_are_rejected_before_any_device_work(cdll):
    one = ctypes.create_string_buffer(512)
    p = ctypes.addressof(one)
    f = cdll.b200fp8_gemm_rowwise
    assert f(None, p, p, p, None, p, 1, 1, 16, 16, 16, 8, p, 512, 0, None) == lib.BAD_ARG
    assert f(p, p, p, p, None, p, 0, 1, 16, 16, 16, 8, p, 512, 0, None) == lib.BAD_ARG
    assert f(p, p, p, p, None, p, 1, 1, 16, 8, 16, 8, p, 512, 0, None) == lib.BAD_ARG  # ldx < K
    assert f(p, p, p, p, None, p, 1 << 40, 1, 16, 16, 16, 8, p, 512, 0, None) == lib.TOO_LARGE
    assert cdll.b200fp8_workspace_init(None, 1024, None) == lib.BAD_ARG
    assert cdll.b200fp8_query_status(None, None) == lib.BAD_ARG


def test_workspace_sizes_and_plans_need_no_device(cdll):
    assert cdll.b200fp8_workspace_bytes(8192, 8192, 8192, 0) == lib.WORKSPACE_HEADER_BYTES
    assert cdll.b200fp8_workspace_bytes(16, 28672, 8192, 0) == lib.WORKSPACE_HEADER_BYTES  # partial sums stay on chip
    skinny = cdll.b200fp8_workspace_bytes(16, 28672, 8192, lib.VARIANT_SKINNY)
    assert skinny > 256 * 1024  # counters + partial sums
    assert cdll.b200fp8_workspace_bytes(0, 1, 1, 0) == 0
    assert cdll.b200fp8_workspace_bytes(256, 256, 256, lib.VARIANT_SKINNY) == 0  # M > 128
    assert lib.describe_plan(8192, 8192, 8192).startswith("tc_2cta")
    assert lib.describe_plan(300, 512, 512).startswith("tc_splitk")  # 6 tiles of 128x256: far too few for 148 SMs
    assert lib.describe_plan(16, 28672, 8192).startswith("tc_splitk tile=128x")
    long_k = lib.describe_plan(16, 2304, 16384)  # few tiles, long K: K is split inside a cluster
    assert long_k.startswith("tc_splitk") and "cluster=1 " not in long_k
    assert lib.describe_plan(16, 1 << 20, 1024).startswith("skinny")  # thousands of tiles: persistent stream-K
    assert lib.describe_plan(100, 1 << 20, 1024).startswith("tc_1cta")
    assert lib.describe_plan(16, 28672, 8192, lib.VARIANT_SKINNY).startswith("skinny")
    forced = lib.describe_plan(16, 4096, 4096, lib.VARIANT_TC_SPLITK | lib.flag_splitk_config(64, 4))
    assert forced.startswith("tc_splitk tile=128x64x128 cluster=4")
    assert lib.describe_plan(16, 28672, 8192, lib.VARIANT_SIMT).startswith("simt")
    # 80 pair tiles would leave most of a second wave empty: one wave of 320-column tiles instead
    assert lib.describe_plan(1000, 5120, 3584).startswith("tc_splitk tile=128x320x128 cluster=1")


def test_rasterisation_group_height_follows_the_shape(cdll):
    """16 row tiles per group when their X panel (16 x tile rows x K bytes) is at most 36 MB and M has a full group."""
    import re

    group = lambda *shape: int(re.search(r"group_m=(\d+)", lib.describe_plan(*shape)).group(1))  # noqa: E731
    assert group(8192, 8192, 8192) == 16 and group(65536, 8192, 8192) == 16 and group(4096, 14336, 4096) == 16
    assert group(16384, 8192, 13312) == 8 and group(16384, 4096, 16384) == 8  # 54 and 67 MB X panels
    assert group(3000, 7168, 2048) == 8 and group(2048, 8192, 2048) == 8  # fewer than 16 row tiles of 256
    assert group(8192, 8192, 8192, lib.VARIANT_TC_1CTA) == 16 and group(1024, 8192, 8192, lib.VARIANT_TC_1CTA) == 8


def test_overlapped_launches_of_cache_resident_problems_get_a_ring_for_two_ctas_per_sm(cdll):
    import re

    smem = lambda plan: int(re.search(r"smem=(\d+)", plan).group(1))  # noqa: E731
    stages = lambda plan: int(re.search(r"stages=(\d+)", plan).group(1))  # noqa: E731
    for shape in [(128, 8192, 2304), (4, 13312, 2048), (64, 13312, 2048), (16, 4096, 6656)]:  # W of 19-27 MB
        deep, shallow = lib.describe_plan(*shape), lib.describe_plan(*shape, lib.FLAG_PDL)
        assert smem(shallow) <= 227 * 1024 // 2 < smem(deep) and 3 <= stages(shallow) < stages(deep), (shape, deep, shallow)
    for shape in [(16, 28672, 8192), (32, 8192, 13312)]:  # W of 109-235 MB comes from HBM: the deep ring stays
        assert lib.describe_plan(*shape, lib.FLAG_PDL).split(" workspace")[0] == lib.describe_plan(*shape).split(" workspace")[0]


def test_check_maps_statuses_to_python_exceptions(cdll):
    lib.check(lib.OK, "x")
    with pytest.raises(NotImplementedError):
        lib.check(lib.UNSUPPORTED_ALIGNMENT, "x")
    with pytest.raises(lib.B200Fp8Error) as e:
        lib.check(lib.DEVICE_TIMEOUT, "x")
    assert e.value.status == lib.DEVICE_TIMEOUT


def test_no_load_in_the_library_uses_cluster_multicast():
    # no TMA / bulk LOAD in this library may carry cluster multicast; the only multicast token
    # allowed is on tcgen05.commit (an mbarrier arrive)
    src_dir = os.path.join(ROOT, "tritonbench_b200", "csrc")
    for name in os.listdir(src_dir):
        if not name.endswith((".cu", ".cuh", ".h")):
            continue
        for line in open(os.path.join(src_dir, name)):
            if "multicast" in line and "cp.async" in line:
                raise AssertionError(f"{name}: {line.strip()}")


def test_one_tile_per_cluster_plans_are_well_formed_for_any_shape(cdll):
    """Host logic only: for random shapes and every forced cluster size the plan string must describe a tile
    width that the cluster can split into 16-column multiples, at least one stage, a ring that fits, and a
    CTA count equal to tiles x cluster."""
    import random
    import re

    rng = random.Random(7)
    pat = re.compile(r"tc_splitk tile=128x(\d+)x128 cluster=(\d+) .* x_rows=(\d+) stages=(\d+) ctas=(\d+) waves=(\d+) smem=(\d+)")
    for _ in range(400):
        m = rng.choice([1, 3, 8, 16, 31, 64, 100, 128, 300, 777, 2000])
        n = rng.choice([8, 24, 100, 256, 1000, 2304, 4096, 5120, 9000, 13312, 28672, 50000])
        k = rng.choice([16, 128, 144, 400, 1024, 2304, 8192, 16384])
        split = rng.choice([0, 1, 2, 4, 8])
        flags = lib.VARIANT_TC_SPLITK | lib.flag_splitk_config(0, split)
        plan = lib.describe_plan(m, n, k, flags)
        got = pat.match(plan)
        assert got, plan
        bn, s, x_rows, stages, ctas, waves, smem = (int(v) for v in got.groups())
        assert 16 <= bn <= 512 and bn % (16 * s) == 0, plan
        assert bn <= 256 or (s == 1 and bn % 64 == 0), plan  # a wide tile: two halves of whole 32-column steps, no K split
        assert split in (0, s), plan
        assert x_rows == (128 if m >= 128 else (m + 7) // 8 * 8), plan
        assert 1 <= stages <= 14 and stages * (x_rows + bn) * 128 <= 192 * 1024, plan
        assert ctas == ((m + 127) // 128) * ((n + bn - 1) // bn) * s and waves >= 1, plan
        assert smem <= 227 * 1024, plan
        # tensor memory: the CTAs one SM can hold by shared memory never need more than its 512 columns
        tmem_cols = 32 if bn <= 32 else 64 if bn <= 64 else 128 if bn <= 128 else 256 if bn <= 256 else 512
        assert (227 * 1024 // smem) * tmem_cols <= 512, plan
