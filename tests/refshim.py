"""Test helper: the reference engine (installed unmodified under ``oracle/_ref`` by
``oracle/Makefile``) with this library's kernels swapped in at the reference's own function
boundary — the swap a maintainer would make by editing imports.

Every hot-path function of the reference (``flashrec.kernel.sglops`` / ``rms_fp8`` / ``silu_fp8`` /
``qk_rope_kv`` / ``beam_trie`` and ``flashrec.attention.kv_indices``) is replaced by a dispatcher: CUDA
tensors go to the same-named function of ``flashrec_b200``, CPU tensors to the reference's original
(its torch branch, which the reference's tests use as the expected side). The replacement is applied to
every loaded ``flashrec.*`` module, so ``from ... import f`` bindings and private aliases follow.
"""

from __future__ import annotations

import importlib
import importlib.util
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
REF_DIR = ROOT / "oracle" / "_ref"

_SWAPS = {
    "flashrec.kernel.sglops": ("flashrec_b200.kernel.sglops",
                               ["rmsnorm", "fused_add_rmsnorm", "per_token_quant_fp8", "fp8_scaled_mm", "silu_and_mul",
                                "store_kv_cache", "apply_rope_inplace", "apply_rope_and_store_kv"]),
    "flashrec.kernel.rms_fp8": ("flashrec_b200.kernel.rms_fp8",
                                ["rmsnorm_per_token_quant_fp8", "fused_add_rmsnorm_per_token_quant_fp8"]),
    "flashrec.kernel.silu_fp8": ("flashrec_b200.kernel.silu_fp8", ["silu_and_mul_per_token_quant_fp8"]),
    "flashrec.kernel.qk_rope_kv": ("flashrec_b200.kernel.qk_rope_kv", ["fused_qk_norm_rope_store_fp8"]),
    "flashrec.kernel.beam_trie": ("flashrec_b200.kernel.beam_trie",
                                  ["trie_mask_candidates", "trie_advance_nodes", "trie_advance_nodes_batched",
                                   "beam_expand_token_ids", "genrec_mask_topk_expand", "call_genrec_cuda",
                                   "try_load_beam_trie"]),
    "flashrec.attention.kv_indices": ("flashrec_b200.attention", ["gather_kv_indices"]),
    "flashrec.search.select": ("flashrec_b200.search", ["joint_select", "select_final_topk"]),
    "flashrec.search.expand": ("flashrec_b200.search", ["apply_temperature", "gumbel_like"]),
}
_installed = {}


def available() -> bool:
    return (REF_DIR / "flashrec" / "__init__.py").exists()


def _tensors(args, kwargs):
    for x in list(args) + list(kwargs.values()):
        if isinstance(x, torch.Tensor):
            yield x


def _dispatcher(name, ours, theirs):
    def f(*args, **kwargs):
        ts = list(_tensors(args, kwargs))
        if ts and all(t.is_cuda for t in ts):
            return ours(*args, **kwargs)
        if name == "try_load_beam_trie":
            return ours()
        return theirs(*args, **kwargs)

    f.__name__ = name
    f.__wrapped_reference__ = theirs
    return f


def install():
    """Import the reference from ``oracle/_ref`` and swap the kernels in. Idempotent.
    Returns the imported ``flashrec`` package."""
    if not available():
        raise RuntimeError("oracle/_ref is missing: run `make -C oracle` where the reference checkout exists")
    if str(REF_DIR) not in sys.path:
        sys.path.insert(0, str(REF_DIR))
    import flashrec  # noqa: F401

    # everything that binds the functions by value must be loaded before the sweep
    for mod in ("flashrec.layers.linear", "flashrec.layers.norm", "flashrec.layers.rotary", "flashrec.kvcache.pool",
                "flashrec.models.qwen3", "flashrec.search.trie", "flashrec.search.state", "flashrec.search.expand",
                "flashrec.engine.graph", "flashrec.kernel"):
        importlib.import_module(mod)
    replace = {}
    for ref_mod, (our_mod, names) in _SWAPS.items():
        rm, om = importlib.import_module(ref_mod), importlib.import_module(our_mod)
        for name in names:
            if (ref_mod, name) in _installed:
                continue
            theirs = getattr(rm, name)
            new = _dispatcher(name, getattr(om, name), theirs)
            replace[id(theirs)] = (theirs, new)
            _installed[(ref_mod, name)] = new
    if replace:
        for mname, mod in list(sys.modules.items()):
            if mod is None or not (mname == "flashrec" or mname.startswith("flashrec.")):
                continue
            for attr, val in list(vars(mod).items()):
                hit = replace.get(id(val))
                if hit is not None and hit[0] is val:
                    setattr(mod, attr, hit[1])
    return sys.modules["flashrec"]


def load_reference_test_module(stem: str):
    """One of the reference's own test files (copied beside the install), imported under a private name
    after the swap so that its module-level imports bind the dispatchers."""
    install()
    path = REF_DIR / "ref_tests" / f"{stem}.py"
    spec = importlib.util.spec_from_file_location(f"_ref_tests_{stem}", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod
