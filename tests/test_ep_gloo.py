"""Expert-parallel exchange logic on CPU: two gloo ranks, arithmetic supplied by
the CPU oracle through the backend interface of moonshine_b200.ep.  The result
of every rank must equal the single-process oracle layer bit for bit, including
when one rank receives no rows at all."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class OracleBackend:
    """CPU stand-in for NativeBackend: same methods, numpy + oracle arithmetic."""

    def __init__(self, cfg, weights, first, per):
        from oracle import k3_oracle as o
        self.o, self.cfg, self.w, self.first, self.per = o, cfg, weights, first, per

    @staticmethod
    def _u16(t):
        return t.numpy().view(np.uint16)

    def route(self, x):
        o, c = self.o, self.cfg
        logits = o.bf16_gemm(self.w["router_weight"], self._u16(x), c["experts"], c["hidden"])
        ids, w = o.router_topk(logits, self.w["router_bias"], c["top_k"], c["route_scale"])
        return torch.from_numpy(ids.view(np.int32).copy()), torch.from_numpy(w)

    def dispatch(self, ids, tokens, top_k, experts, tag):
        idn = ids.numpy().view(np.uint32).reshape(tokens, top_k)
        off, toks, slots = self.o.group_routes(idn, experts)
        inv = np.empty(tokens * top_k, np.uint32)
        inv[slots] = np.arange(tokens * top_k, dtype=np.uint32)
        t = lambda a: torch.from_numpy(a.view(np.int32).copy())
        return t(off), t(slots), t(toks), t(inv)

    def gather(self, rows, index, tag):
        return rows[index.long()].contiguous()

    def experts(self, rows, offsets_local, index):
        o, c, w = self.o, self.cfg, self.w
        off = offsets_local.numpy()
        x = self._u16(rows[index.long()].contiguous())
        out = np.zeros_like(x)
        for le in range(self.per):
            lo, hi = int(off[le]), int(off[le + 1])
            if lo == hi:
                continue
            e = self.first + le
            g = o.mxfp4_gemm(w["w1_packed"][e], w["w1_scales"][e], x[lo:hi], c["expert_hidden"], c["hidden"])
            u = o.mxfp4_gemm(w["w3_packed"][e], w["w3_scales"][e], x[lo:hi], c["expert_hidden"], c["hidden"])
            a = o.activation(g, u, c["activation"], c["beta"], c["linear_beta"])
            out[lo:hi] = o.mxfp4_gemm(w["w2_packed"][e], w["w2_scales"][e], a, c["hidden"], c["expert_hidden"])
        return torch.from_numpy(out.view(np.int16).copy())

    def shared(self, x):
        o, c, w = self.o, self.cfg, self.w
        s, d = c["shared_hidden"], c["hidden"]
        if not s:
            return None
        xs = self._u16(x)
        g = o.q8_gemm(w["shared_gate_q"], w["shared_gate_s"], xs, s, d, c["q8_block"], c["q8_scale_type"])
        u = o.q8_gemm(w["shared_up_q"], w["shared_up_s"], xs, s, d, c["q8_block"], c["q8_scale_type"])
        a = o.activation(g, u, c["activation"], c["beta"], c["linear_beta"])
        out = o.q8_gemm(w["shared_down_q"], w["shared_down_s"], a, d, s, c["q8_block"], c["q8_scale_type"])
        return torch.from_numpy(out.view(np.int16).copy())

    def combine(self, rows, index, weights, shared, tokens):
        o, c = self.o, self.cfg
        k, d = c["top_k"], c["hidden"]
        picked = self._u16(rows)[index.numpy().view(np.uint32)].reshape(tokens, k, d)
        out = o.weighted_sum(np.ascontiguousarray(picked), weights.numpy(), tokens, k, d)
        if shared is not None:
            out = o.add(out, self._u16(shared))
        return torch.from_numpy(out.view(np.int16).copy())


def _worker(rank, world, port, mode, results):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from moonshine_b200 import ep, synth
        from oracle import k3_oracle as o
        cfg = synth.tiny_config()
        weights = synth.make_layer(cfg, seed=31)
        if mode == "rank1_idle":
            weights["router_bias"][: cfg["experts"] // 2] += np.float32(5.0)   # every route stays on rank 0
        tokens = 24
        x = synth.activations(31, tokens, cfg["hidden"])
        want, want_ids, _, _, _ = o.moe_layer(weights, x)
        first, per = ep.shard_range(cfg["experts"], world, rank)
        backend = OracleBackend(cfg, weights, first, per)
        lo, hi = rank * tokens // world, (rank + 1) * tokens // world
        xl = torch.from_numpy(x[lo:hi].view(np.int16).copy())
        if mode == "pipelined":
            # three row ranges advancing in lock step, each with its own backend
            backends = [OracleBackend(cfg, weights, first, per) for _ in range(3)]
            out, ids, _ = ep.ep_forward_pipelined(backends, xl, cfg)
        elif mode == "row_per_route":
            out, ids, _ = ep.ep_forward(backend, xl, cfg, once_per_destination=False)
        else:
            out, ids, _ = ep.ep_forward(backend, xl, cfg, once_per_destination=True)
        got = out.numpy().view(np.uint16)
        ok = np.array_equal(got, want[lo:hi]) and np.array_equal(ids.numpy().view(np.uint32), want_ids[lo:hi])
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode,world", [("balanced", 2), ("rank1_idle", 2), ("balanced", 4), ("pipelined", 2),
                                        ("row_per_route", 2)])
def test_expert_parallel_ranks_equal_single_process(mode, world, oracle):
    port = 29600 + (os.getpid() % 200) + {"balanced": 0, "rank1_idle": 1, "pipelined": 5, "row_per_route": 7}[mode] + 2 * world
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_worker, args=(world, port, mode, results), nprocs=world, join=True)
        assert dict(results) == {r: True for r in range(world)}


def test_exchange_plan():
    from moonshine_b200 import ep
    # 2 ranks, 4 experts (2 per rank); counts[source, expert]
    counts = torch.tensor([[3, 0, 2, 1], [1, 2, 0, 4]], dtype=torch.int64)
    send, recv, starts, lengths, off = ep.exchange_plan(counts, 1, 2, 2)       # rank 1 owns experts 2, 3
    assert send == [3, 4] and recv == [3, 4]
    # received rows: source 0 -> [e2, e2, e3], source 1 -> [e3 x 4]; grouped: e2 (s0 x2, s1 x0), e3 (s0 x1, s1 x4)
    assert starts.tolist() == [0, 3, 2, 3] and lengths.tolist() == [2, 0, 1, 4]
    assert off.tolist() == [0, 2, 7]
    send, recv, starts, lengths, off = ep.exchange_plan(counts, 0, 0, 2)
    assert send == [3, 3] and recv == [3, 3] and off.tolist() == [0, 4, 6]


def test_exchange_form_by_world_size():
    from moonshine_b200 import ep
    assert ep.rows_once_per_destination(2, 16) and ep.rows_once_per_destination(4, 16)
    assert not ep.rows_once_per_destination(8, 16)
    assert not ep.rows_once_per_destination(2, 2)


def test_destination_splits():
    from moonshine_b200 import ep
    offsets = torch.tensor([0, 2, 2, 5, 9, 9, 9, 10, 12], dtype=torch.int32)
    assert ep.destination_splits(offsets, 8, 2) == [9, 3]
    assert ep.destination_splits(offsets, 8, 4) == [2, 7, 0, 3]
    assert ep.shard_range(896, 8, 3) == (336, 112)
    with pytest.raises(ValueError):
        ep.shard_range(10, 4, 0)


def c_plan(offsets_all, world, rank, experts):
    import ctypes as C
    from moonshine_b200 import _native
    per = experts // world
    u32 = lambda n: (C.c_uint32 * n)()
    flat = (C.c_uint32 * offsets_all.size)(*offsets_all.ravel().tolist())
    send, recv, brs, bds, br, off = u32(world), u32(world), u32(per * world), u32(per * world), u32(per * world), u32(per + 1)
    assert _native.lib().k3_moe_ep_plan(flat, world, rank, experts, send, recv, brs, bds, br, off)
    return [list(a) for a in (send, recv, brs, bds, br, off)]


@pytest.mark.parametrize("world,experts", [(2, 4), (4, 16), (8, 896)])
def test_library_plan_matches_python_plan_and_regroups_to_single_gpu_order(world, experts):
    """k3_moe_ep_plan (the host step of the C entry point) against ep.exchange_plan, and the
    property the layer relies on: reading the received rows through the plan's blocks gives
    the single-GPU grouping order (expert asc, global route asc)."""
    from moonshine_b200 import ep
    rng = np.random.default_rng(world)
    per, tokens_per_rank, k = experts // world, 9, min(4, experts)
    ids = np.stack([rng.permutation(experts)[:k] for _ in range(world * tokens_per_rank)]).astype(np.uint32)
    if world == 4:
        ids[ids >= 12] = 0                        # the last rank receives nothing at all
    counts = np.zeros((world, experts), np.int64)
    offsets_all = np.zeros((world, experts + 1), np.uint32)
    for r in range(world):
        local = ids[r * tokens_per_rank:(r + 1) * tokens_per_rank]
        counts[r] = np.bincount(local.ravel(), minlength=experts)
        offsets_all[r, 1:] = np.cumsum(counts[r])
    for rank in range(world):
        send, recv, brs, bds, br, off = c_plan(offsets_all, world, rank, experts)
        psend, precv, starts, lengths, poff = ep.exchange_plan(torch.from_numpy(counts), rank, rank * per, per)
        assert send == psend and recv == precv and off == poff.tolist()
        assert brs == starts.tolist() and br == lengths.tolist()
        assert bds == (np.cumsum(lengths.numpy()) - lengths.numpy()).tolist()
        # emulate: what each source sends (its routes sorted expert asc, route asc, restricted to
        # this rank's experts), concatenated source by source, then read through the blocks
        received = []
        for s in range(world):
            local = ids[s * tokens_per_rank:(s + 1) * tokens_per_rank].ravel()
            routes = np.arange(local.size) + s * tokens_per_rank * k           # global route numbers
            order = np.lexsort((routes, local))
            keep = [(int(local[i]), int(routes[i])) for i in order if rank * per <= local[i] < (rank + 1) * per]
            received += keep
        grouped = [None] * len(received)
        for b in range(per * world):
            for i in range(br[b]):
                grouped[bds[b] + i] = received[brs[b] + i]
        assert grouped == sorted(received)                                      # expert asc, global route asc
        assert off[-1] == len(received)
