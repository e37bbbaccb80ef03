"""Per-layer-embedding store: table file, read plan (hits / misses / runs), LRU row cache, IO budget, gather."""
import pytest
import torch

from tensorrt_edge_llm_b200.runtime import native as rt
from tensorrt_edge_llm_b200.runtime.ple import PleStore, write_ple_table


@pytest.fixture()
def table(tmp_path):
    t = torch.randn(300, 4 * 8).to(torch.float16)
    p = str(tmp_path / "ple.bin")
    write_ple_table(p, t, layers=4)
    return p, t


def test_plan_hits_misses_and_runs(table):
    path, _ = table
    tb = rt.PleTable(path)
    assert (tb.rows, tb.row_bytes, tb.layers, tb.dtype) == (300, 64, 4, 0)
    cache = rt.PleCache(8)
    p = cache.plan([10, 11, 12, 50, 11, 200], tb.row_bytes)
    assert (p.hits, p.misses, p.deferred) == (0, 5, 0) and p.slots[1] == p.slots[4]          # a repeated id shares its slot
    assert [(r.first_row, r.count, r.staging_row) for r in p.runs] == [(10, 3, 0), (50, 1, 3), (200, 1, 4)]
    assert p.bytes == 5 * 64 and sorted(p.miss_rows) == p.miss_rows
    p2 = cache.plan([11, 12, 13], tb.row_bytes)
    assert (p2.hits, p2.misses) == (2, 1) and p2.slots[0] == p.slots[1]
    # eviction takes the least recently used rows and never one the step itself uses
    p3 = cache.plan([100, 101, 102, 103, 104, 11], tb.row_bytes)
    assert p3.misses == 5 and cache.lookup(11) >= 0 and cache.lookup(12) >= 0 and cache.lookup(10) < 0
    small = rt.PleCache(2)
    p4 = small.plan([1, 2, 3], tb.row_bytes)
    assert p4.misses == 2 and p4.deferred == 1 and p4.slots[2] == -1                         # more distinct rows than slots
    with pytest.raises(RuntimeError):
        rt.PleTable(path + ".missing")


def test_store_gather_matches_table_and_budget_defers(table):
    path, t = table
    store = PleStore(path, cache_rows=64)
    ids = [5, 6, 7, 299, 5, 0]
    got = store.gather(ids)
    assert got.shape == (6, 4, 8) and torch.equal(got.view(6, -1), t[ids])
    again = store.gather([7, 6, 150])
    assert torch.equal(again.view(3, -1), t[[7, 6, 150]]) and store.cache.hits == 2 and 0 < store.hit_rate < 1
    # cache churn: every row still comes back right after eviction
    g = torch.Generator().manual_seed(0)
    for _ in range(20):
        ids = torch.randint(0, 300, (40,), generator=g).tolist()
        assert torch.equal(store.gather(ids).view(40, -1), t[ids])
    # an IO budget of two rows per step (burst of two steps): the rest is deferred and arrives on later steps
    tight = PleStore(path, cache_rows=64, io_bytes_per_step=128)
    first = tight.gather([20, 21, 22, 23, 24, 25]).view(6, -1)
    assert tight.deferred_rows == 2 and torch.equal(first[:4], t[20:24]) and (first[4:] == 0).all()
    second = tight.gather([24, 25]).view(2, -1)
    assert torch.equal(second, t[24:26])


def test_bfloat16_table(tmp_path):
    t = torch.randn(16, 2 * 4).to(torch.bfloat16)
    p = str(tmp_path / "b.bin")
    write_ple_table(p, t, layers=2)
    s = PleStore(p, cache_rows=4)
    assert s.dtype == torch.bfloat16 and torch.equal(s.gather([3, 9]).view(2, -1), t[[3, 9]])
