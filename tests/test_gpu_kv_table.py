"""Slot-table bookkeeping of a decode tick on the GPU (through the C ABI) against the fixture made
with the reference's own remap_by_parents / write_decode / gather_kv_indices /
copy_prefill_to_beams_many, against the CPU oracle on random waves, and at the bench's size."""

import numpy as np
import pytest
import torch

from conftest import load_golden
from oracle import sid_oracle as O
from test_oracle_golden import _kv_table_replay

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _gpu_step(table, rows, gi, sl, new_slot, parents, prefix, capacity=None):
    from flashrec_b200.attention import kv_table_step

    n = int(rows.numel())
    total = int(sl.sum())
    out = torch.full((total if capacity is None else capacity,), -7, dtype=torch.int32, device=DEV)
    indptr = torch.empty(n + 1, dtype=torch.int32, device=DEV)
    d = lambda t, dt: None if t is None else t.to(device=DEV, dtype=dt).contiguous()
    kv_table_step(table, d(rows, torch.int64), d(sl, torch.int32), out, indptr, new_slot=d(new_slot, torch.int64),
                  parents_rel=d(parents, torch.int64), prefix_len=d(prefix, torch.int32),
                  group_indptr=d(gi, torch.int32))
    return indptr.cpu(), out.cpu()


def test_kv_table_ticks_golden():
    from flashrec_b200.attention import copy_prefill_to_beams_many

    g = load_golden("kv_table")
    table = torch.from_numpy(g["table0"].copy()).to(DEV)
    step = lambda t, rows, gi, sl, ns, par, pre: _gpu_step(t, rows, gi, sl, ns, par, pre)[1]
    fan = lambda t, srcs, beam_rows, m: copy_prefill_to_beams_many(t, srcs.to(DEV), beam_rows.to(DEV).contiguous(), m)
    for tag, tab, flat in _kv_table_replay(g, step, fan, table):
        if tag == "fanout":
            assert np.array_equal(tab.cpu().numpy(), g["table_fanout"])
        else:
            assert np.array_equal(tab.cpu().numpy(), g[f"table{tag + 1}"]), tag
            assert np.array_equal(flat.numpy(), g[f"flat{tag}"]), tag


def test_remap_known_answer_and_identity():
    # tests/test_kv_remap.py:19-37 of the reference: window 2:4 gathered by parents; no new column
    table = torch.arange(20, dtype=torch.int32).view(4, 5).clone().to(DEV)
    rows, gi = torch.arange(4), torch.tensor([0, 4])
    sl, pre = torch.full((4,), 4, dtype=torch.int32), torch.full((4,), 2, dtype=torch.int32)
    indptr, flat = _gpu_step(table, rows, gi, sl, None, torch.tensor([0, 0, 1, 1]), pre)
    t = table.cpu()
    assert t[:, 2:4].tolist() == [[2, 3], [2, 3], [7, 8], [7, 8]]
    assert t[:, :2].tolist() == [[0, 1], [5, 6], [10, 11], [15, 16]] and t[:, 4].tolist() == [4, 9, 14, 19]
    assert indptr.tolist() == [0, 4, 8, 12, 16] and flat.view(4, 4).tolist() == t[:, :4].tolist()
    before = table.clone()
    _gpu_step(table, rows, gi, sl, None, torch.arange(4), pre)
    assert torch.equal(table, before)


@pytest.mark.parametrize("n_req,bw,max_prompt,ticks", [(5, 16, 40, 4), (3, 1, 9, 2), (32, 512, 1024, 3), (2, 2048, 300, 4)])
def test_kv_table_random_waves_vs_oracle(n_req, bw, max_prompt, ticks):
    rng = np.random.default_rng(n_req * 1000 + bw)
    plens = rng.integers(1, max_prompt + 1, n_req)
    n = n_req * bw
    max_seq = int(plens.max()) + ticks
    table_h = torch.from_numpy(rng.integers(1, 1 << 30, (n + 3, max_seq)).astype(np.int32))
    rows = torch.from_numpy(rng.permutation(n + 3)[:n].astype(np.int64))
    gi = torch.arange(n_req + 1, dtype=torch.int32) * bw
    prefix = torch.from_numpy(np.repeat(plens, bw).astype(np.int32))
    table_d = table_h.clone().to(DEV)
    parents = None
    for tick in range(ticks):
        sl = prefix + tick + 1
        new_slot = torch.from_numpy(rng.integers(1, 1 << 30, n).astype(np.int64))
        ref_indptr, ref_flat = O.kv_table_step(table_h, rows, gi, sl, new_slot, parents, prefix)
        indptr, flat = _gpu_step(table_d, rows, gi, sl, new_slot, parents, prefix)
        assert torch.equal(indptr, ref_indptr) and torch.equal(flat, ref_flat), tick
        assert torch.equal(table_d.cpu(), table_h), tick
        # properties that hold at any size: every row ends in its new slot and keeps its prompt
        last = flat[(indptr[1:] - 1).long()]
        assert torch.equal(last.long(), new_slot)
        kind = tick % 3  # forks, a permutation, out-of-range values (clamped)
        if kind == 0:
            parents = torch.from_numpy(rng.integers(0, bw, n).astype(np.int64))
        elif kind == 1:
            parents = torch.from_numpy(np.concatenate([rng.permutation(bw) for _ in range(n_req)]).astype(np.int64))
        else:
            parents = torch.from_numpy(rng.integers(-3, bw + 3, n).astype(np.int64))


def test_plain_gather_and_empty():
    from flashrec_b200.attention import kv_table_step

    table = torch.arange(60, dtype=torch.int32).view(6, 10).to(DEV)
    before = table.clone()
    rows, sl = torch.tensor([4, 0, 5]), torch.tensor([3, 0, 10], dtype=torch.int32)
    indptr, flat = _gpu_step(table, rows, None, sl, None, None, None)
    assert torch.equal(table, before)  # without parents and new slots the table is only read
    assert indptr.tolist() == [0, 3, 3, 13] and flat.tolist() == [40, 41, 42] + list(range(50, 60))
    # zero rows: a no-op
    e64, e32 = torch.empty(0, dtype=torch.int64, device=DEV), torch.empty(0, dtype=torch.int32, device=DEV)
    kv_table_step(table, e64, e32, e32, torch.zeros(1, dtype=torch.int32, device=DEV))
    # a list buffer that is too short drops the tail from the list and from the table update, nothing else
    table2 = before.clone()
    gi = torch.tensor([0, 3])
    from flashrec_b200 import device_status

    assert device_status() == (0, 0)
    _gpu_step(table2, rows, gi, sl, torch.tensor([7, 8, 9]), None, None, capacity=3)
    assert table2[4, 2].item() == 7 and table2[5, 9].item() == before[5, 9].item()
    # ... and the overflow is reported through the status word (read-and-clear)
    assert device_status() == (-1, 41)
    assert device_status() == (0, 0)


def test_parent_outside_the_table_keeps_the_rows_own_window():
    from flashrec_b200.attention import kv_table_step

    table = torch.arange(40, dtype=torch.int32).view(4, 10).to(DEV)
    before = table.clone()
    # batch rows 0, 1 are table rows 1 and 99 (99 does not exist); both name the other as parent
    rows = torch.tensor([1, 99], device=DEV)
    sl = torch.tensor([6, 6], dtype=torch.int32, device=DEV)
    pre = torch.tensor([2, 2], dtype=torch.int32, device=DEV)
    par = torch.tensor([1, 0], device=DEV)
    gi = torch.tensor([0, 2], dtype=torch.int32, device=DEV)
    out = torch.full((12,), -7, dtype=torch.int32, device=DEV)
    indptr = torch.zeros(3, dtype=torch.int32, device=DEV)
    kv_table_step(table, rows, sl, out, indptr, new_slot=torch.tensor([70, 71], device=DEV), parents_rel=par,
                  prefix_len=pre, group_indptr=gi)
    want = before.clone()
    want[1, 5] = 70
    assert torch.equal(table, want)  # row 1 kept its own window: its parent has no table row
    assert out[:6].tolist() == [10, 11, 12, 13, 14, 70]


def test_type_errors():
    from flashrec_b200.attention import copy_prefill_to_beams_many, kv_table_step

    table = torch.zeros((4, 8), dtype=torch.int32, device=DEV)
    rows = torch.arange(4, device=DEV)
    sl = torch.ones(4, dtype=torch.int32, device=DEV)
    out, indptr = torch.zeros(4, dtype=torch.int32, device=DEV), torch.zeros(5, dtype=torch.int32, device=DEV)
    with pytest.raises(TypeError):
        kv_table_step(table.long(), rows, sl, out, indptr)
    with pytest.raises(TypeError):  # parents without prefix_len / group_indptr
        kv_table_step(table, rows, sl, out, indptr, parents_rel=rows)
    with pytest.raises(ValueError):
        copy_prefill_to_beams_many(table, rows[:1], rows.view(1, 4), 9)


def test_rows_outside_the_table_and_overlong_lengths_are_skipped_or_clamped():
    from flashrec_b200.attention import kv_table_step

    table = torch.arange(40, dtype=torch.int32).view(4, 10).to(DEV)
    before = table.clone()
    rows = torch.tensor([1, 99, -3, 2], device=DEV)          # two rows that do not exist
    sl = torch.tensor([4, 3, 2, 25], dtype=torch.int32, device=DEV)  # the last one longer than the table is wide
    out = torch.full((34,), -7, dtype=torch.int32, device=DEV)
    indptr = torch.empty(5, dtype=torch.int32, device=DEV)
    new_slot = torch.tensor([500, 501, 502, 503], device=DEV)
    kv_table_step(table, rows, sl, out, indptr, new_slot=new_slot)
    assert indptr.tolist() == [0, 4, 7, 9, 34]
    t = table.cpu()
    assert t[1, 3].item() == 500 and t[2, 9].item() == 503  # clamped to the last column of the table
    t[1, 3], t[2, 9] = before[1, 3], before[2, 9]
    assert torch.equal(t, before.cpu())                      # nothing else was touched
    o = out.cpu()
    assert o[:4].tolist() == [10, 11, 12, 500] and o[9:19].tolist() == list(range(20, 29)) + [503]
