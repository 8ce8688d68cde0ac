"""Kernel-level entry points, same names as the reference's ``flashrec.kernel``
package (kernel/__init__.py:1-19)."""

from flashrec_b200.kernel.beam_trie import (
    GenrecFusedResult,
    GenrecFusedWorkspace,
    beam_expand_token_ids,
    call_genrec_cuda,
    genrec_mask_topk_expand,
    trie_advance_nodes,
    trie_mask_candidates,
    try_load_beam_trie,
)

__all__ = [
    "GenrecFusedResult",
    "GenrecFusedWorkspace",
    "beam_expand_token_ids",
    "call_genrec_cuda",
    "genrec_mask_topk_expand",
    "trie_advance_nodes",
    "trie_mask_candidates",
    "try_load_beam_trie",
]
