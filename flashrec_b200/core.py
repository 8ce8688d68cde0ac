"""Data carriers of the decode path, field for field as the reference defines them:
``ForwardBatch`` (core.py:81-101) and ``ExpandCaptureSpec`` (engine/graph.py:46-56).

Objects of the reference's own classes are accepted wherever these are (the code reads
attributes, it does not test types)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch


@dataclass
class ForwardBatch:
    """One forward; ``n_rows`` = total beam rows (decode) or prompts (prefill) (core.py:81-101).

    The fields and their order are the reference's; everything after ``seq_lens`` has a default so
    that callers of this library may leave out what its kernels do not need (``seq_lens_cpu`` is only
    used to size the attention scratch without a device read). Two additions at the end:
    ``qo_indptr`` (int32, device, ``[n_rows + 1]``), the running sum of ``extend_seq_lens`` that the
    prefill attention reads — derived from ``extend_seq_lens`` when absent.

    Prefill (``is_prefill``): ``input_ids`` / ``positions`` / ``out_cache_loc`` hold one entry per
    extend token, ``seq_lens`` / ``kv_indptr`` one per request; ``extend_seq_lens`` and
    ``extend_prefix_lens`` are host lists."""

    input_ids: torch.Tensor
    req_pool_indices: Optional[torch.Tensor]
    seq_lens: torch.Tensor
    seq_lens_cpu: Optional[torch.Tensor] = None
    positions: Optional[torch.Tensor] = None
    out_cache_loc: Optional[torch.Tensor] = None
    is_prefill: bool = False
    extend_prefix_lens: Optional[List[int]] = None
    extend_seq_lens: Optional[List[int]] = None
    kv_indices: Optional[torch.Tensor] = None  # ragged slot ids, page size 1
    kv_indptr: Optional[torch.Tensor] = None
    buffers_ready: bool = False  # decode graph static buffers already filled
    want_expand: bool = False
    qo_indptr: Optional[torch.Tensor] = None

    @property
    def n_rows(self) -> int:
        return int(self.seq_lens.numel())


@dataclass
class ExpandCaptureSpec:
    """What a decode graph needs to capture the row top-k + fused trie expand after the head
    (engine/graph.py:46-56): beam width, candidates per beam, winners per request, token-plane
    width, the candidate token ids and the dense trie tables (or a ``DeviceTrie`` in
    ``allow_table`` with ``next_node`` None: CSR and bitmap catalogs take the same fused step)."""

    beam_width: int
    cand: int
    select_k: int
    width: int
    cand_ids: torch.Tensor
    allow_table: object
    next_node: Optional[torch.Tensor]
    token_base: int
    invalid_node: int
