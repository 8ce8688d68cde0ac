"""ctypes binding of ``libflashrec_b200.so`` (the C ABI in ``include/flashrec_b200.h``).

The library is the product path: there is no CPU or eager fallback. If the
shared object is missing, or a kernel reports a non-zero status, the caller
gets an exception.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p, POINTER
from pathlib import Path
from typing import Optional

import torch

# FLASHREC_B200_LIB selects another build of the same library (e.g. to compare two builds in one process
# launch each); by default the library built in-tree next to this file is loaded.
_LIB_PATH = Path(os.environ.get("FLASHREC_B200_LIB") or Path(__file__).resolve().parent / "libflashrec_b200.so").resolve()
_lib: Optional[ctypes.CDLL] = None

FR_OK = 0
_STATUS_NAMES = {
    0: "FR_OK",
    -1: "FR_ERR_BAD_ARG",
    -2: "FR_ERR_UNSUPPORTED",
    -3: "FR_ERR_CUDA",
    -4: "FR_ERR_TIMEOUT",
}


class FlashRecKernelError(RuntimeError):
    """A C-ABI entry point returned a non-zero status."""

    def __init__(self, fn: str, status: int):
        self.fn = fn
        self.status = int(status)
        super().__init__(f"{fn} failed: {_STATUS_NAMES.get(int(status), status)}")


class FrTrie(ctypes.Structure):
    """Mirror of ``struct fr_trie`` (include/flashrec_b200.h)."""

    _fields_ = [
        ("kind", ctypes.c_int32),
        ("next_is_i32", ctypes.c_int32),
        ("allow", c_void_p),
        ("next", c_void_p),
        ("csr_keys", c_void_p),
        ("csr_child", c_void_p),
        ("n_edges", c_int64),
        ("bitmap", c_void_p),
        ("child_base", c_void_p),
        ("level_off", c_void_p),
        ("words_per_node", ctypes.c_int32),
        ("reserved_", ctypes.c_int32),
        ("n_rows", c_int64),
        ("vsz", c_int64),
        ("token_base", c_int64),
        ("invalid_node", c_int64),
    ]


FR_TRIE_NONE, FR_TRIE_DENSE, FR_TRIE_CSR, FR_TRIE_BITMAP = 0, 1, 2, 3

P = c_void_p
_I = c_int
_L = c_int64
_F = c_float

# name -> argtypes (restype is always int unless listed in _RESTYPES)
_SIGNATURES = {
    "fr_version": [],
    "fr_device_status": [POINTER(c_int), POINTER(c_int)],
    "fr_rms_quant_fp8": [P, P, P, _F, P, P, _I, _I, P],
    "fr_rmsnorm_bf16": [P, P, P, _F, P, _I, _I, P],
    "fr_token_quant_fp8": [P, _I, P, P, _I, _I, P],
    "fr_silu_mul_quant_fp8": [P, P, P, _I, _I, P],
    "fr_silu_mul_bf16": [P, P, _I, _I, P],
    "fr_gemm_fp8_w8a8": [P, P, P, P, P, P, _I, _I, _I, _I, _L, _L, _L, _I, P],
    "fr_gemm_fp8_w8a8_add": [P, P, P, P, P, _I, _I, _I, _L, _L, _L, _I, P],
    "fr_gemm_fp8_qkv_rope": [P, P, P, P, P, _L, _I, _I, _I, _I, _I, _L, _L, P, P, P, P, _F, P, _I, P, P, _L, _L, _L, _L, _I,
                             P],
    "fr_gemm_fp8_silu_mul": [P, P, P, P, P, P, _I, _I, _I, _L, _L, _L, _I, P],
    "fr_quant_known_amax_fp8": [P, P, P, P, _I, _I, P],
    "fr_qk_norm_rope_kv_fp8": [P, P, P, _L, _L, _L, _L, _L, _L, P, P, P, P, _F, P, _I, P, P, _L, _L, _L, _L, _I,
                               _I, _I, _I, _I, P],
    "fr_rope_neox_inplace": [P, P, P, _L, _L, _L, _L, _L, _L, P, P, P, _I, P, P, _L, _L, _L, _L, _I, _I, _I, _I, _I, P],
    "fr_store_kv_fp8": [P, P, _L, _L, _L, _L, P, P, P, _L, _L, _L, _L, _I, _I, _I, _I, _I, P],
    "fr_gather_kv_indices": [P, _L, P, P, P, P, _I, _I, P],
    "fr_kv_table_step": [P, _L, _I, _I, P, P, _I, P, P, P, P, P, P, _I, _I, P],
    "fr_kv_table_fanout": [P, _L, _I, P, P, _I, _I, _I, P],
    "fr_embedding_bf16": [P, P, P, _I, _I, _I, P],
    "fr_decode_attn_plan": [P, P, P, _I, _I, P, P],
    "fr_decode_attn_scratch_bytes": [_I, _I, _I],
    "fr_trie_build_workspace_bytes": [_L],
    "fr_trie_build_csr": [P, _L, _I, P, P, P, _L, P, P, _L, P],
    "fr_trie_csr_to_bitmap": [P, P, _L, _I, P, P, P, P, P, _I, P],
    "fr_decode_attn_fp8": [P, _L, _L, P, P, _L, _L, _L, _L, P, P, P, P, P, _L, _I, _I, _I, _I, _I, _I, _I, _F, P, _L,
                           _I, P],
    "fr_prefill_attn_fp8": [P, _L, _L, P, P, _L, _L, _L, _L, P, P, P, P, _L, _I, _I, _I, _I, _I, _I, _I, _I, _F, P, _L,
                            P],
    "fr_decode_attn_reuse_fp8": [P, _L, _L, P, P, _L, _L, _L, _L, P, P, P, P, P, _L, _I, _I, _I, _I, _I, _I, _I, _F, P,
                                 _L, _I, P, P],
    "fr_logsumexp_rows": [P, _L, P, P, P, _L, _I, _I, P],
    "fr_topk_rows": [P, _L, P, P, P, P, _I, _I, _I, P],
    "fr_lse_combine_shards": [P, P, P, P, _I, _I, _L, P],
    "fr_trie_mask": [P, P, P, P, P, _F, _L, _L, P],
    "fr_trie_advance": [P, P, P, P, P, _I, _I, _I, P],
    "fr_beam_expand": [P, P, P, P, _I, _I, _I, _I, P],
    "fr_mask_topk_expand": [P] * 16 + [_I] * 8 + [P],
    "fr_mask_topk_expand_static": [P] * 15 + [_I] * 8 + [P],
    "fr_sid_beam_step": [P] * 7 + [_L] + [P] * 9 + [_L] * 3 + [_I] * 7 + [P],
    "fr_joint_select_workspace_bytes": [_I, _I],
    "fr_joint_select": [P] * 8 + [P, P, P, P, P, _I, P, _L, _I, _I, _I, _I, P],
    "fr_select_final_topk": [P] * 4 + [P, P, P, P, _I, _I, _I, _I, P],
    "fr_sid_head_topk_workspace_bytes": [_I, _I, _I, _I],
    "fr_sid_head_topk": [P] * 6 + [P, P, _L, P, P, _L, _I] + [P] * 8 + [_L] * 3 + [_I] * 8 + [P, P, P, _L, _I, P],
    "fr_topk_merge_shards": [P] * 16 + [_L] * 2 + [_I] * 7 + [P],
}
_RESTYPES = {"fr_version": c_char_p, "fr_decode_attn_scratch_bytes": c_int64,
             "fr_sid_head_topk_workspace_bytes": c_int64, "fr_joint_select_workspace_bytes": c_int64,
             "fr_trie_build_workspace_bytes": c_int64}


def lib_path() -> Path:
    return _LIB_PATH


def load() -> ctypes.CDLL:
    """Load the shared library (once). Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        raise FlashRecKernelError(
            f"load({_LIB_PATH}): not built; run `python -m flashrec_b200.build`", -3
        )
    lib = ctypes.CDLL(str(_LIB_PATH))
    for name, argtypes in _SIGNATURES.items():
        fn = getattr(lib, name, None)
        if fn is None:
            continue  # checked by tests against include/flashrec_b200.h
        fn.argtypes = argtypes
        fn.restype = _RESTYPES.get(name, c_int)
    _lib = lib
    return lib


def stream_ptr(device: Optional[torch.device] = None) -> int:
    """Raw cudaStream_t of torch's current stream."""
    return torch.cuda.current_stream(device).cuda_stream


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def call(name: str, *args) -> None:
    """Call an int-status entry point; raise on non-zero status."""
    fn = getattr(load(), name)
    st = fn(*args)
    if st != FR_OK:
        raise FlashRecKernelError(name, st)


def device_status() -> tuple[int, int]:
    """Read-and-clear the device status word: (code, site). Synchronises."""
    code = c_int(0)
    site = c_int(0)
    call("fr_device_status", ctypes.byref(code), ctypes.byref(site))
    return code.value, site.value


def require_cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise FlashRecKernelError("flashrec_b200 (tensor not on a CUDA device: no CPU path)", -1)
