"""The C-ABI library builds for sm_100a, loads, and exports every symbol the header declares."""

import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "tensorfold_b200.h"


def declared_symbols() -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(tf_[a-z0-9_]+)\s*\(", text)))


def test_header_and_loader_agree(lib):
    from tensorfold_b200 import _lib

    names = declared_symbols()
    assert names, "no declarations found in the header"
    assert set(names) == set(_lib.SIGNATURES), set(names) ^ set(_lib.SIGNATURES)
    for name in names:
        assert isinstance(getattr(lib.cdll, name), ctypes._CFuncPtr)


def test_pure_host_entry_points(lib):
    assert lib.tf_version() >= 1000
    assert lib.tf_qmm_workers() == 148
    # 16-column x 64-k records of 576 bytes (group 64) / 640 bytes (group 32): 4.5 and 5 bits a weight
    assert lib.tf_qmm_tiled_bytes(17408, 5120, 64) == 17408 * 5120 * 9 // 16
    assert lib.tf_qmm_tiled_bytes(768, 2048, 32) == 768 * 2048 * 5 // 8
    assert lib.tf_qmm_tiled_bytes(40, 64, 64) == 16 * 576         # columns padded to a 256-column block
    assert lib.tf_packed_bytes(8, 5120, 64) == 80 * 8 * 132 and lib.tf_packed_bytes(9, 2048, 32) == 32 * 16 * 136
    assert lib.tf_qmm_tiled_bytes(16, 100, 64) == 0               # K must be a multiple of 64
    assert lib.tf_qmm_scratch_bytes() > 16384


def test_bad_arguments_are_refused_before_any_launch(lib):
    from tensorfold_b200 import _lib

    buf = (ctypes.c_char * 4096)()
    p = ctypes.addressof(buf)
    p = (p + 255) & ~255
    big = lib.tf_qmm_scratch_bytes()
    assert lib.tf_qmm(p, p, p, p, big, 0, 64, 64, 64, 0, None, None) == _lib.TF_EINVAL      # no rows
    assert lib.tf_qmm(p, p, p, p, big, 129, 64, 64, 64, 0, None, None) == _lib.TF_EINVAL    # too many rows
    assert lib.tf_qmm(p, p, p, p, big, 8, 64, 96, 64, 0, None, None) == _lib.TF_EINVAL      # K % 64
    assert lib.tf_qmm(p, p, p, p, big, 8, 64, 64, 16, 0, None, None) == _lib.TF_EINVAL      # group
    assert lib.tf_qmm(p + 2, p, p, p, big, 8, 64, 64, 64, 0, None, None) == _lib.TF_EALIGN
    assert lib.tf_qmm(p, p, p, None, big, 8, 64, 64, 64, 0, None, None) == _lib.TF_ESCRATCH
    assert lib.tf_qmm(p, p, p, p, 16, 8, 64, 64, 64, 0, None, None) == _lib.TF_ESCRATCH


def test_k_schedule_is_a_function_of_shape_only():
    from tensorfold_b200 import lane_qmm

    segs = lane_qmm.segments(17408, 5120)
    assert len(segs) == 68                # 256-column blocks
    for cb in segs:                      # segments tile [0, 80) k tiles in order, no gaps
        assert cb[0][0] == 0 and cb[-1][1] == 80
        assert all(a[1] == b[0] for a, b in zip(cb, cb[1:]))
    assert lane_qmm.split_k(17408, 5120) == max(len(c) for c in segs)
    assert lane_qmm.split_k(48, 5120) >= 8      # a narrow projection is cut along K to fill the GPU


def test_product_has_no_oracle_or_cpu_path():
    pkg = ROOT / "tensorfold_b200"
    for path in pkg.rglob("*.py"):
        text = path.read_text()
        assert "oracle" not in text.replace("no CPU or PyTorch fallback", ""), path
