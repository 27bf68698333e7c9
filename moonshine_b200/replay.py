"""Decode-routes traces as workload drivers.

The reference's ``--decode-diagnostics PREFIX`` writes ``PREFIX.routes.csv`` with
the header ``capture,step,position,layer,observed_hit_mask,expert_0,...,expert_15``
(docs/observability.md:57-70), one line per routed layer and decode step
(k3_engine.cu:1622-1644): which 16 experts the router chose, in rank order, and
which of them were resident in the layer's slot cache (bit r = expert_r).
Routed layers are numbered from 1.

This module reads and writes that format, generates seeded traces of the same
shape (skewed expert popularity plus step-to-step reuse) for machines without a
recorded trace, and replays a trace three ways:

* ``replay_cache``  through the slot policy: hit masks as the reference would
  have logged them for a given slot count, admissions and bytes read;
* ``ep_load``       onto an expert-parallel partition: assignments per rank and
  step, the imbalance an all-to-all of that step would see;
* ``replay_store``  through a ``PartialStore`` on the GPU: every line's experts
  are admitted as the policy decides and their products run out of the slots.
"""
from __future__ import annotations

import csv

import numpy as np

from .store import SlotCache

TOP_K = 16
HEADER = ["capture", "step", "position", "layer", "observed_hit_mask"] + [f"expert_{r}" for r in range(TOP_K)]


class Routes:
    """Columns of a trace as arrays: capture, step u64; position, layer, hit_mask
    u32 [lines]; experts u16 [lines, 16]."""

    def __init__(self, capture, step, position, layer, hit_mask, experts):
        self.capture = np.asarray(capture, dtype=np.uint64)
        self.step = np.asarray(step, dtype=np.uint64)
        self.position = np.asarray(position, dtype=np.uint32)
        self.layer = np.asarray(layer, dtype=np.uint32)
        self.hit_mask = np.asarray(hit_mask, dtype=np.uint32)
        self.experts = np.asarray(experts, dtype=np.uint16).reshape(-1, TOP_K)
        n = len(self.capture)
        for name in ("step", "position", "layer", "hit_mask", "experts"):
            if len(getattr(self, name)) != n:
                raise ValueError(f"column {name} has {len(getattr(self, name))} entries, capture has {n}")

    def __len__(self):
        return len(self.capture)


def write_routes(path: str, routes: Routes) -> None:
    with open(path, "w", newline="") as f:
        w = csv.writer(f, lineterminator="\n")
        w.writerow(HEADER)
        for i in range(len(routes)):
            w.writerow([int(routes.capture[i]), int(routes.step[i]), int(routes.position[i]),
                        int(routes.layer[i]), int(routes.hit_mask[i])] + [int(e) for e in routes.experts[i]])


def read_routes(path: str, experts: int | None = None) -> Routes:
    """Parse a routes file.  Rejects a wrong header, short or non-numeric lines,
    repeated experts within a line (the slot policy refuses such a batch,
    k3_expert_cache.c:139-147) and, when ``experts`` is given, ids out of range."""
    cols = [[] for _ in range(5)]
    ids = []
    with open(path, newline="") as f:
        reader = csv.reader(f)
        header = next(reader, None)
        if header != HEADER:
            raise ValueError(f"{path}: not a decode-routes file (header {header})")
        for number, row in enumerate(reader, start=2):
            if len(row) != len(HEADER):
                raise ValueError(f"{path}:{number}: {len(row)} fields, expected {len(HEADER)}")
            try:
                values = [int(v) for v in row]
            except ValueError:
                raise ValueError(f"{path}:{number}: non-numeric field") from None
            line_ids = values[5:]
            if len(set(line_ids)) != TOP_K:
                raise ValueError(f"{path}:{number}: repeated expert id")
            if min(line_ids) < 0 or (experts is not None and max(line_ids) >= experts) or max(line_ids) > 0xFFFF:
                raise ValueError(f"{path}:{number}: expert id out of range")
            for c, v in zip(cols, values[:5]):
                c.append(v)
            ids.append(line_ids)
    return Routes(*cols, np.array(ids, dtype=np.uint16).reshape(-1, TOP_K))


def synthetic_routes(steps: int, layers: int, experts: int = 896, seed: int = 0, zipf_s: float = 1.1,
                     reuse: float = 0.5, capture: int = 1, first_position: int = 0) -> Routes:
    """A seeded trace of ``steps`` decode steps over ``layers`` routed layers.
    Per layer the experts have a fixed Zipf popularity (exponent ``zipf_s``, a
    different permutation per layer); a step keeps each expert of the layer's
    previous step with probability ``reuse`` and draws the rest by popularity.
    hit masks are left 0 (``replay_cache`` fills them for a slot count)."""
    rng = np.random.default_rng(seed)
    rank_weight = 1.0 / np.arange(1, experts + 1) ** zipf_s
    popularity = []
    for _ in range(layers):
        p = np.empty(experts)
        p[rng.permutation(experts)] = rank_weight
        popularity.append(p / p.sum())
    previous = [None] * layers
    cap, stp, pos, lay, ids = [], [], [], [], []
    for step in range(steps):
        for layer in range(layers):
            keep = []
            if previous[layer] is not None:
                keep = [int(e) for e in previous[layer] if rng.random() < reuse]
            p = popularity[layer].copy()
            p[keep] = 0.0
            fresh = rng.choice(experts, size=TOP_K - len(keep), replace=False, p=p / p.sum())
            chosen = np.array(keep + [int(e) for e in fresh], dtype=np.int64)
            # rank order = router order: by popularity, as a stand-in for the score
            chosen = chosen[np.argsort(-popularity[layer][chosen], kind="stable")]
            previous[layer] = chosen
            cap.append(capture)
            stp.append(step)
            pos.append(first_position + step)
            lay.append(layer + 1)
            ids.append(chosen)
    return Routes(cap, stp, pos, lay, np.zeros(len(cap), dtype=np.uint32), np.array(ids, dtype=np.uint16))


def replay_cache(routes: Routes, slots_per_layer: int, bytes_per_expert: int = 17_547_264,
                 first_layer: int = 1) -> dict:
    """Replay every line through the slot policy, in file order.

    -> {"hit_mask": u32 [lines], "admissions": u32 [lines], "mismatches": lines
    whose mask differs from the file's observed_hit_mask, "stats": policy
    telemetry, "physical_read_bytes": bytes_per_expert per miss (the reference's
    ledger counts the aligned span per miss, k3_engine.cu:1615-1621; the default
    is the real checkpoint's span size), "hit_rate"}.
    A trace recorded by the reference with the same slot count and a cold start
    replays with zero mismatches."""
    layers = int(routes.layer.max()) - first_layer + 1 if len(routes) else 1
    cache = SlotCache(layers, slots_per_layer)
    masks = np.zeros(len(routes), dtype=np.uint32)
    admitted = np.zeros(len(routes), dtype=np.uint32)
    try:
        for i in range(len(routes)):
            masks[i], admitted[i] = cache.replay_line(int(routes.layer[i]) - first_layer, routes.experts[i])
        stats = cache.stats()
    finally:
        cache.close()
    return {
        "hit_mask": masks,
        "admissions": admitted,
        "mismatches": int(np.count_nonzero(masks != routes.hit_mask)),
        "stats": stats,
        "physical_read_bytes": int(stats["misses"]) * bytes_per_expert,
        "hit_rate": stats["hits"] / max(1, stats["accesses"]),
    }


def ep_load(routes: Routes, world: int, experts: int = 896) -> dict:
    """Assignments per expert-parallel rank (contiguous experts/world per rank, the
    partition of ``moonshine_b200.ep``) for every line, and per decode step summed
    over the layers.  "imbalance" = busiest rank / mean, the factor by which the
    slowest rank of an all-to-all step exceeds a perfectly even one."""
    if experts % world:
        raise ValueError("experts must divide evenly over the ranks")
    owner = routes.experts.astype(np.int64) // (experts // world)
    per_line = np.stack([(owner == r).sum(axis=1) for r in range(world)], axis=1)
    totals = per_line.sum(axis=0)
    mean = TOP_K / world
    return {
        "per_line": per_line,
        "totals": totals,
        "line_imbalance_mean": float((per_line.max(axis=1) / mean).mean()) if len(routes) else 0.0,
        "line_imbalance_max": float(per_line.max() / mean) if len(routes) else 0.0,
        "total_imbalance": float(totals.max() / max(1e-9, totals.mean())),
    }


def replay_store(stores: dict, routes: Routes, x, weights, first_layer: int = 1) -> dict:
    """Run every line's experts on the GPU out of the layers' slot tables.
    ``stores`` maps a trace layer number to its ``PartialStore``; lines of other
    layers are skipped.  ``x`` bf16 [1, d] and ``weights`` f32 [16] are reused for
    every line (a trace carries no activations).  -> hit masks of the lines run,
    bytes admitted, and the last output."""
    masks, out = [], None
    for i in range(len(routes)):
        store = stores.get(int(routes.layer[i]))
        if store is None:
            continue
        out, mask = store.token(x, routes.experts[i], weights)
        masks.append(mask)
    return {"hit_mask": np.array(masks, dtype=np.uint32),
            "bytes_admitted": sum(s.bytes_admitted for s in stores.values()), "last": out}
