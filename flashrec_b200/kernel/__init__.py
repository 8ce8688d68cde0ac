"""Kernel-level entry points under the names the reference's ``flashrec.kernel`` package exports
(kernel/__init__.py:1-19), so that ``from flashrec_b200.kernel import genrec_mask_topk_expand`` reads like the
reference's import. Everything comes from :mod:`flashrec_b200.kernel.beam_trie`."""

from flashrec_b200.kernel import beam_trie as _bt

__all__ = sorted(
    name for name in (
        "GenrecFusedResult GenrecFusedWorkspace beam_expand_token_ids call_genrec_cuda genrec_mask_topk_expand "
        "trie_advance_nodes trie_mask_candidates try_load_beam_trie"
    ).split()
)
globals().update({name: getattr(_bt, name) for name in __all__})
