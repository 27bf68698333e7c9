"""Regenerates tests/golden/slot_cache.npz from the reference's own slot policy:

    make -C oracle ref REF=<reference tree>
    python tests/golden/make_slot_cache_golden.py

oracle/_ref/libk3expertcache_ref.so is the reference's k3_expert_cache.c compiled
as it is.  Seeded call sequences (plan / commit / abort / invalidate over several
layers, including slot counts below the batch size) are run through it and every
answer is stored: per plan the hit and admit flags and both slot numbers, after
every commit the layer's LRU order, at the end the telemetry.  The product's
slot cache must reproduce all of it (tests/test_store.py).
"""
import ctypes as C
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from moonshine_b200.store import SlotCache          # noqa: E402

CASES = [  # (slots per layer, experts per plan, experts, steps, seed)
    (24, 16, 64, 300, 1),
    (16, 16, 40, 300, 2),
    (8, 16, 30, 200, 3),
    (32, 16, 896, 300, 4),
    (5, 3, 9, 200, 5),
]
LAYERS = 3
OP_PLAN_COMMIT, OP_PLAN_ABORT, OP_INVALIDATE = 0, 1, 2


def script(case):
    """The seeded call sequence of a case: (op, layer, ids | (first, count))."""
    cap, n, experts, steps, seed = case
    rng = np.random.default_rng(seed)
    calls = []
    for _ in range(steps):
        layer = int(rng.integers(0, LAYERS))
        ids = rng.choice(experts, size=n, replace=False).astype(np.uint16)
        calls.append((OP_PLAN_ABORT if rng.random() < 0.1 else OP_PLAN_COMMIT, layer, ids))
        if rng.random() < 0.05:
            first = int(rng.integers(0, LAYERS * cap))
            count = int(rng.integers(1, LAYERS * cap - first + 1))
            calls.append((OP_INVALIDATE, 0, (first, count)))
    return calls


def run(cache, calls, cap):
    """-> (accesses i64 [plans, n, 4], snapshots i32 [plans, cap] (-1 padded), stats)."""
    accesses, snaps = [], []
    for op, layer, arg in calls:
        if op == OP_INVALIDATE:
            cache.invalidate_slots(*arg)
            continue
        accesses.append([[int(h), int(a), s, d] for h, a, s, d in cache.plan(layer, arg)])
        if op == OP_PLAN_ABORT:
            cache.abort(layer)
        else:
            cache.commit(layer)
        snap = cache.snapshot(layer)
        snaps.append(snap + [-1] * (cap - len(snap)))
    st = cache.stats()
    return (np.array(accesses, dtype=np.int64), np.array(snaps, dtype=np.int32),
            np.array([st[k] for k in ("batches", "accesses", "hits", "misses", "admissions", "evictions")],
                     dtype=np.int64))


def main():
    ref = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libk3expertcache_ref.so"))
    out = {}
    for index, case in enumerate(CASES):
        cache = SlotCache(LAYERS, case[0], handle=ref, prefix="k3_expert_cache_")
        acc, snaps, stats = run(cache, script(case), case[0])
        cache.close()
        out[f"case{index}_accesses"] = acc
        out[f"case{index}_snapshots"] = snaps
        out[f"case{index}_stats"] = stats
    path = os.path.join(HERE, "slot_cache.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
