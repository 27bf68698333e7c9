"""Slot policy of the partially resident store and the decode-routes replay (host
code, no GPU).  The policy is checked against answers recorded from the
reference's own k3_expert_cache.c (tests/golden/slot_cache.npz, see
make_slot_cache_golden.py) and, where that file's build is present
(oracle/_ref), against it live; error behaviour follows k3_expert_cache.c."""
import ctypes as C
import os

import numpy as np
import pytest

from moonshine_b200 import build, replay
from moonshine_b200.store import SlotCache, StoreError, pack_spans, span_layout
from tests.golden import make_slot_cache_golden as gold

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libk3expertcache_ref.so")


@pytest.fixture(scope="module", autouse=True)
def native():
    build.build()


@pytest.mark.parametrize("index", range(len(gold.CASES)))
def test_policy_reproduces_reference_answers(index):
    case = gold.CASES[index]
    want = np.load(os.path.join(ROOT, "tests", "golden", "slot_cache.npz"))
    cache = SlotCache(gold.LAYERS, case[0])
    acc, snaps, stats = gold.run(cache, gold.script(case), case[0])
    np.testing.assert_array_equal(acc, want[f"case{index}_accesses"])
    np.testing.assert_array_equal(snaps, want[f"case{index}_snapshots"])
    np.testing.assert_array_equal(stats, want[f"case{index}_stats"])


@pytest.mark.skipif(not os.path.exists(REF_LIB), reason="reference slot policy not built on this machine")
def test_policy_matches_reference_build_live():
    ref = C.CDLL(REF_LIB)
    rng = np.random.default_rng(11)
    mine, theirs = SlotCache(4, 20), SlotCache(4, 20, handle=ref, prefix="k3_expert_cache_")
    for _ in range(600):
        layer = int(rng.integers(0, 4))
        ids = rng.choice(48, size=int(rng.integers(1, 25)), replace=False)
        assert mine.plan(layer, ids) == theirs.plan(layer, ids)
        mine.commit(layer)
        theirs.commit(layer)
        assert mine.snapshot(layer) == theirs.snapshot(layer)
    assert mine.stats() == theirs.stats()


def test_error_behaviour():
    # texts and conditions of k3_expert_cache.c:79-83, 128-147, 256-262, 311-327, 341-352, 370-389
    with pytest.raises(StoreError, match="invalid expert-cache dimensions"):
        SlotCache(0, 4)
    with pytest.raises(StoreError, match="invalid expert-cache dimensions"):
        SlotCache(2, 0)
    c = SlotCache(2, 4)
    with pytest.raises(StoreError, match="invalid expert-cache plan arguments"):
        c.plan(2, [1, 2])
    with pytest.raises(StoreError, match="invalid expert-cache plan arguments"):
        c.plan(0, [])
    with pytest.raises(StoreError, match="duplicate IDs"):
        c.plan(0, [1, 2, 1])
    with pytest.raises(StoreError, match="no pending plan"):
        c.commit(0)
    c.plan(0, [1, 2])
    with pytest.raises(StoreError, match="already has a pending plan"):
        c.plan(0, [3])
    with pytest.raises(StoreError, match="invalid expert-cache snapshot request"):
        c.snapshot(0)
    with pytest.raises(StoreError, match="cannot reset expert cache with a pending plan"):
        c.reset()
    with pytest.raises(StoreError, match="cannot invalidate expert cache with a pending plan"):
        c.invalidate_slots(0, 1)
    c.plan(1, [5])                      # one pending plan per layer, layers are independent
    c.abort(1)
    c.abort(0)
    c.abort(0)                          # aborting nothing is not an error
    assert c.stats()["batches"] == 0    # aborted plans leave no trace
    with pytest.raises(StoreError, match="invalid expert-cache invalidation range"):
        c.invalidate_slots(0, 0)
    with pytest.raises(StoreError, match="invalid expert-cache invalidation range"):
        c.invalidate_slots(7, 2)
    assert c.slot_count() == 8
    assert c.storage_bytes(17_547_264) == 8 * 17_547_264
    assert c.storage_bytes(1 << 62) == (1 << 64) - 1


def test_plan_commit_semantics():
    c = SlotCache(1, 4)
    first = c.plan(0, [10, 11, 12])
    assert [a[:2] for a in first] == [(False, True)] * 3
    assert [a[3] for a in first] == [0, 1, 2]                 # lowest free slots, oldest entry first
    c.abort(0)
    assert c.snapshot(0) == []                                # a plan alone does not touch the live state
    assert c.plan(0, [10, 11, 12]) == first
    c.commit(0)
    assert c.snapshot(0) == [10, 11, 12]
    second = c.plan(0, [12, 13, 14])
    assert second[0] == (True, False, 2, 0xFFFFFFFF)          # hit: read from its slot until commit
    # 10 is evicted; free slots go to the new entries oldest first, lowest slot first
    assert second[1][:2] == (False, True) and second[1][3] == 0
    assert second[2][:2] == (False, True) and second[2][3] == 3
    c.commit(0)
    assert c.snapshot(0) == [11, 12, 13, 14]
    # more experts than slots: the early misses fall out again and are not admitted
    big = c.plan(0, [20, 21, 22, 23, 24, 25])
    assert [a[1] for a in big] == [False, False, True, True, True, True]
    c.commit(0)
    st = c.stats()
    assert (st["batches"], st["accesses"], st["hits"], st["misses"]) == (3, 12, 1, 11)
    c.reset()
    assert c.snapshot(0) == [] and c.stats()["accesses"] == 0


def test_span_layout_matches_the_checkpoint():
    offsets, total = span_layout(3584, 3072)
    assert offsets == [0, 5_505_024, 5_849_088, 11_354_112, 11_698_176, 17_203_200]
    assert total == 17_547_264
    w = {name: np.full((2, 8), i, dtype=np.uint8) for i, name in enumerate(
        ("w1_packed", "w1_scales", "w2_packed", "w2_scales", "w3_packed", "w3_scales"))}
    w["w1_packed"] = np.zeros((2, 64 * 32 // 2), dtype=np.uint8)
    w["w3_packed"] = np.full((2, 64 * 32 // 2), 4, dtype=np.uint8)
    w["w2_packed"] = np.full((2, 64 * 32 // 2), 2, dtype=np.uint8)
    for name, v in (("w1_scales", 1), ("w2_scales", 3), ("w3_scales", 5)):
        w[name] = np.full((2, 64 * 32 // 32), v, dtype=np.uint8)
    spans = pack_spans(w, 2, 64, 32)
    off, size = span_layout(64, 32)
    assert spans.shape == (2, size)
    for i, o in enumerate(off):
        assert spans[1, o] == i and spans[1, (off + [size])[i + 1] - 1] == i


def test_routes_round_trip_and_validation(tmp_path):
    routes = replay.synthetic_routes(steps=12, layers=3, experts=896, seed=4)
    assert len(routes) == 36 and set(routes.layer) == {1, 2, 3}
    assert all(len(set(line)) == 16 for line in routes.experts.tolist())
    path = str(tmp_path / "x.routes.csv")
    replay.write_routes(path, routes)
    assert open(path).readline().strip() == (
        "capture,step,position,layer,observed_hit_mask," + ",".join(f"expert_{r}" for r in range(16)))
    back = replay.read_routes(path, experts=896)
    for name in ("capture", "step", "position", "layer", "hit_mask", "experts"):
        np.testing.assert_array_equal(getattr(back, name), getattr(routes, name))
    lines = open(path).read().splitlines()
    for bad, message in (
        (["capture,step"] + lines[1:], "not a decode-routes file"),
        (lines[:1] + [lines[1] + ",7"], "fields"),
        (lines[:1] + [lines[1].replace(",", ",x", 1)], "non-numeric"),
        (lines[:1] + [",".join(lines[1].split(",")[:-1] + [lines[1].split(",")[5]])], "repeated expert"),
        (lines[:1] + [",".join(lines[1].split(",")[:-1] + ["900"])], "out of range"),
    ):
        p = str(tmp_path / "bad.csv")
        open(p, "w").write("\n".join(bad) + "\n")
        with pytest.raises(ValueError, match=message):
            replay.read_routes(p, experts=896)


def test_cache_replay_reproduces_logged_hit_masks(tmp_path):
    # a trace whose masks were logged with 32 slots replays with no mismatch at 32
    # slots and with mismatches at another slot count
    routes = replay.synthetic_routes(steps=40, layers=4, experts=896, seed=9, reuse=0.6)
    logged = replay.replay_cache(routes, 32)
    assert logged["mismatches"] > 0                       # the synthetic file holds zeros
    routes.hit_mask = logged["hit_mask"]
    path = str(tmp_path / "t.routes.csv")
    replay.write_routes(path, routes)
    again = replay.replay_cache(replay.read_routes(path), 32)
    assert again["mismatches"] == 0
    assert again["stats"]["accesses"] == 40 * 4 * 16
    assert again["physical_read_bytes"] == again["stats"]["misses"] * 17_547_264
    assert replay.replay_cache(routes, 16)["mismatches"] > 0
    # every first access of a layer is a miss; hits need reuse
    assert logged["hit_mask"][:4].tolist() == [0, 0, 0, 0]
    assert 0.2 < logged["hit_rate"] < 0.95
    bigger = replay.replay_cache(routes, 64)
    assert bigger["hit_rate"] >= logged["hit_rate"]


def test_ep_load_counts():
    routes = replay.synthetic_routes(steps=20, layers=2, experts=896, seed=2)
    load = replay.ep_load(routes, 8)
    assert load["per_line"].shape == (40, 8)
    assert (load["per_line"].sum(axis=1) == 16).all()
    assert load["totals"].sum() == 40 * 16
    manual = np.zeros(8, dtype=np.int64)
    for line in routes.experts:
        for e in line:
            manual[int(e) // 112] += 1
    np.testing.assert_array_equal(load["totals"], manual)
    assert load["line_imbalance_max"] >= load["line_imbalance_mean"] >= 1.0
    with pytest.raises(ValueError):
        replay.ep_load(routes, 5)
