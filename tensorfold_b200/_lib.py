"""ctypes binding of ``libtensorfold_b200.so`` (the C ABI in ``include/tensorfold_b200.h``).

There is no fallback: if the library is missing, importing a kernel wrapper raises. Tensors cross
the boundary as raw device pointers; the stream is torch's current stream.
"""

from __future__ import annotations

import ctypes
from ctypes import c_double, c_float, c_int, c_longlong, c_size_t, c_ulonglong, c_void_p
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libtensorfold_b200.so"

TF_OK, TF_EINVAL, TF_EALIGN, TF_ESCRATCH, TF_ECUDA, TF_ESTALL = 0, -1, -2, -3, -4, -5
_NAMES = {TF_EINVAL: "TF_EINVAL (unsupported shape, size or flag)", TF_EALIGN: "TF_EALIGN (misaligned pointer)",
          TF_ESCRATCH: "TF_ESCRATCH (scratch missing or too small)", TF_ECUDA: "TF_ECUDA (launch refused)",
          TF_ESTALL: "TF_ESTALL (a bounded device wait ran out)"}

# name -> (restype, argtypes); the single list the loader, the tests and the header must agree on
SIGNATURES: dict[str, tuple] = {
    "tf_version": (c_int, []),
    "tf_qmm_workers": (c_int, []),
    "tf_qmm_scratch_bytes": (c_size_t, []),
    "tf_packed_bytes": (c_size_t, [c_int, c_int, c_int]),
    "tf_qmm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_int, c_int, c_int, c_int,
                       c_void_p, c_void_p]),
    "tf_qmm_set_trace": (c_int, [c_void_p]),
    "tf_qmm_next": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_int, c_int, c_int, c_int,
                            c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "tf_qmm_grouped": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_size_t, c_int,
                               c_int, c_int, c_int, c_void_p, c_void_p]),
    "tf_pack_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "tf_qmm_tiled_bytes": (c_size_t, [c_int, c_int, c_int]),
    "tf_qmm_tile": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "tf_qmm_untile": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "tf_packed_tc_bytes": (c_size_t, [c_int, c_int, c_int]),
    "tf_qmm_tc_tiled_bytes": (c_size_t, [c_int, c_int, c_int]),
    "tf_qmm_tc": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_int, c_int, c_int, c_int,
                          c_void_p, c_void_p]),
    "tf_pack_rows_tc": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "tf_qmm_tc_set_trace": (c_int, [c_void_p]),
    "tf_repack_tc": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "tf_qmm_tc_tile": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "tf_qmm_tc_untile": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "tf_norm_xs": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                           c_int, c_int, c_float, c_void_p]),
    "tf_swiglu": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "tf_gated_norm": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                              c_float, c_void_p]),
    "tf_gate_mul": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "tf_attn_prep": (c_int, [c_void_p, c_size_t, c_void_p, c_size_t, c_void_p, c_size_t, c_void_p, c_void_p, c_void_p,
                             c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p]),
    "tf_gdn_pre": (c_int, [c_void_p, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t,
                           c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                           c_int, c_int, c_void_p]),
    "tf_embed": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "tf_gdn_chain": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                             c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "tf_gdn_fused": (c_int, [c_void_p, c_size_t, c_void_p, c_size_t, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p, c_void_p,
                             c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                             c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]),
    "tf_gdn_replay": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                              c_longlong, c_longlong, c_longlong, c_longlong, c_int, c_int, c_int, c_int, c_void_p]),
    "tf_conv_commit": (c_int, [c_void_p, c_size_t, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_int,
                               c_int, c_void_p]),
    "tf_attention_scratch_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "tf_attention_chunks": (c_int, [c_int]),
    "tf_lane_attention_paged_gated": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                              c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_int, c_void_p,
                                              c_size_t, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p,
                                              c_void_p]),
    "tf_lane_attention_paged": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                        c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_int, c_int, c_int,
                                        c_int, c_int, c_int, c_float, c_void_p]),
    "tf_lane_attention_paged_static": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                               c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                               c_float, c_void_p]),
    "tf_kv_commit": (c_int, [c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p,
                             c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "tf_moe_max_problems": (c_int, [c_int, c_int, c_int]),
    "tf_moe_router": (c_int, [c_void_p, c_size_t, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "tf_moe_select": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "tf_moe_group": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                             c_void_p, c_void_p, c_void_p]),
    "tf_moe_slot_bytes": (c_size_t, [c_int, c_int]),
    "tf_moe_push": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_size_t, c_int, c_int, c_void_p, c_void_p]),
    "tf_moe_combine_peer": (c_int, [c_void_p, c_size_t, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p,
                                    c_void_p, c_void_p]),
    "tf_moe_pack": (c_int, [c_void_p, c_size_t, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p]),
    "tf_moe_act": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p]),
    "tf_moe_combine": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p]),
    "tf_peer_slot_bytes": (c_size_t, [c_int, c_int, c_int]),
    "tf_peer_exchange": (c_int, [c_void_p, c_int, c_int, c_void_p, c_size_t, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                 c_void_p]),
    "tf_qmm_act": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int,
                           c_int, c_void_p, c_void_p]),
    "tf_swiglu_tiled": (c_int, [c_void_p, c_size_t, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "tf_qmm_peer": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p,
                            c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "tf_norm_xs_peer": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                c_int, c_int, c_float, c_void_p, c_size_t, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "tf_set_poll_limit": (None, [ctypes.c_uint]),
    "tf_topk_scratch_bytes": (c_size_t, [c_int, c_int, c_int]),
    "tf_topk_rows": (c_int, [c_void_p, c_size_t, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "tf_sample_rows": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_ulonglong, c_double, c_int, c_double, c_void_p,
                               c_int, c_void_p]),
}

_lib = None
_launches = 0          # kernel-launching entry points called so far (what a CUDA graph of a step holds)
_NO_LAUNCH = {"tf_version", "tf_qmm_set_trace", "tf_qmm_tc_set_trace", "tf_set_poll_limit", "tf_qmm_workers", "tf_qmm_scratch_bytes", "tf_packed_bytes", "tf_qmm_tiled_bytes",
              "tf_attention_scratch_bytes", "tf_attention_chunks", "tf_packed_tc_bytes", "tf_qmm_tc_tiled_bytes", "tf_topk_scratch_bytes", "tf_moe_max_problems", "tf_moe_slot_bytes", "tf_peer_slot_bytes"}


def launch_count() -> int:
    return _launches


class _Counted:
    """A bound entry point that counts successful kernel launches (the paged attention and the top-k queue two each)."""

    def __init__(self, fn, n):
        self.fn, self.n = fn, n

    def __call__(self, *args):
        global _launches
        rc = self.fn(*args)
        if rc == 0:
            _launches += self.n
        return rc



def load() -> ctypes.CDLL:
    """The kernel library, loaded once. Raises if it has not been built."""

    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(f"{LIB_PATH} is missing: run `python -m tensorfold_b200.build` "
                               "(there is no CPU or PyTorch fallback for the lane kernels)")
        lib = ctypes.CDLL(str(LIB_PATH))
        class Bound:
            pass

        bound = Bound()
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
            setattr(bound, name, fn if name in _NO_LAUNCH else _Counted(fn, 2 if name.startswith("tf_lane_attention_paged") or name == "tf_topk_rows" else 1))
        bound.cdll = lib
        _lib = bound
    return _lib


def check(code: int, what: str) -> None:
    if code != TF_OK:
        err = ValueError if code in (TF_EINVAL, TF_EALIGN, TF_ESCRATCH) else RuntimeError
        raise err(f"{what}: {_NAMES.get(code, code)}")


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def need_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("lane kernels take CUDA tensors only (there is no CPU path)")


class Status:
    """The device status word kernels report a run-out bounded wait to; read at sync points."""

    def __init__(self, device):
        self.word = torch.zeros(1, dtype=torch.int32, device=device)

    def raise_if_set(self) -> None:
        code = int(self.word.item())
        if code:
            self.word.zero_()
            raise RuntimeError(f"a lane kernel reported {_NAMES.get(code, code)}")


_status: dict[int, Status] = {}


def status(device) -> Status:
    idx = torch.device(device).index or 0
    if idx not in _status:
        _status[idx] = Status(device)
    return _status[idx]
