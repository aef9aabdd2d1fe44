"""Recipe for the reference's own CUDA lane path as a checker on the GPU box.

Test infrastructure only: the files it produces live under ``oracle/_ref/`` (git-ignored, never
committed, never imported by the package) and are read by ``tests/test_reference_gpu.py`` and by the
optional ``reference_gpu`` leg of ``bench.py``. It copies, unmodified, the few source files of the
reference's Triton/CUDA lane path from a checkout of the reference (the path given, or the default below) into a
package skeleton, so that ``import tensorfold.families.qwen3_5.cuda.qmm`` works where the checkout does
not exist. Nothing is built here: the Triton kernels compile on first use and the gdn kernels
(``gdn_tree.cu`` / ``gdn.cu``) are JIT-built by the reference's own loader.

    python oracle/make_ref.py [/path/to/reference]
"""

from __future__ import annotations

import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"

# package skeleton: empty __init__ files (the reference's own family __init__ modules import the whole
# engine); then the lane-path modules themselves
DENSE = ["qmm.py", "qmm_fast.py", "glue.py", "attention.py", "forward.py", "weights.py", "gdn_tree.py", "gdn_tree.cpp",
         "gdn_tree.cu", "reference.py", "sampling.py", "distributed.py"]
MOE = ["qmm.py", "moe.py", "glue.py", "gdn.py", "gdn.cpp", "gdn.cu", "attention.py"]
ENGINE = ["exact_sampling.py"]


def make(reference: Path = Path("/root/reference")) -> Path | None:
    src = reference / "src" / "tensorfold"
    if not src.is_dir():
        return None
    if OUT.exists():
        shutil.rmtree(OUT)
    pkg = OUT / "tensorfold"
    for sub in ("", "families", "families/qwen3_5", "families/qwen3_5/cuda", "families/qwen4_exp", "families/qwen4_exp/cuda",
                "engine"):
        d = pkg / sub
        d.mkdir(parents=True, exist_ok=True)
        (d / "__init__.py").write_text("")
    for name in DENSE:
        shutil.copyfile(src / "families" / "qwen3_5" / "cuda" / name, pkg / "families" / "qwen3_5" / "cuda" / name)
    for name in MOE:
        shutil.copyfile(src / "families" / "qwen4_exp" / "cuda" / name, pkg / "families" / "qwen4_exp" / "cuda" / name)
    for name in ENGINE:
        shutil.copyfile(src / "engine" / name, pkg / "engine" / name)
    return OUT


if __name__ == "__main__":
    made = make(Path(sys.argv[1]) if len(sys.argv) > 1 else Path("/root/reference"))
    print(made if made else "no reference checkout found: nothing made")
