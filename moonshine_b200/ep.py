"""Expert-parallel routed-MoE layer over ``torch.distributed``.

Partitioning: tokens data-parallel (rank r owns the contiguous rows
[r*T/G, (r+1)*T/G)), experts expert-parallel (rank g holds the contiguous
experts [g*E/G, (g+1)*E/G) in its HBM slot table).  Router, top-k and the
shared expert are computed where the token lives.  Per layer there is one
exchange step each way:

  1. route + dispatch on the source: rows sorted (expert asc, route asc); the
     rows for destination g are one contiguous slice because experts are
     contiguous per rank;
  2. one all-gather of every rank's per-expert row counts (the only host read of
     the pass: it gives each rank its send and receive splits and the layout of
     what it will receive), then the all-to-all of the bf16 rows themselves
     (``all_to_all_single`` with uneven splits) - each token row once per
     destination, however many of its routes go there, with a 4-byte slot per
     route telling the destination which received row the route reads;
  3. on the destination the received rows (source rank asc, expert asc, route asc)
     are regrouped (expert asc, source rank asc, route asc) - with the contiguous
     token partition this is exactly the single-GPU grouping order - through a
     gather index built from the count matrix, folded into the grouped expert
     products on the local shard;
  4. rows go back through the inverse permutation and the reverse all-to-all;
  5. combine on the source in rank order (same arithmetic as one GPU).

The arithmetic is delegated to a *backend*: ``NativeBackend`` calls the CUDA
library; tests pass a CPU backend to exercise this file's exchange logic with
``gloo`` ranks.  No collective is used beyond the all-gather and the two all-to-alls above.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist

from . import ops, synth
from .layer import MoELayer


def shard_range(experts: int, world: int, rank: int) -> tuple[int, int]:
    if experts % world != 0:
        raise ValueError("expert count must divide evenly over the ranks")
    per = experts // world
    return rank * per, per


def destination_splits(offsets: torch.Tensor, experts: int, world: int) -> list[int]:
    """Rows this rank sends to each destination, from the expert offsets [E+1]."""
    per = experts // world
    bounds = offsets[::per][: world + 1].to("cpu", torch.int64)
    return [int(bounds[g + 1] - bounds[g]) for g in range(world)]


class NativeBackend:
    """Arithmetic on the GPU through the C-ABI (one MoELayer holding the shard)."""

    def __init__(self, layer: MoELayer):
        self.layer = layer
        self.cfg = layer.cfg
        self.device = layer.device
        self._bufs = {}

    def _buf(self, name, shape, dtype):
        t = self._bufs.get(name)
        n = int(np.prod(shape))
        if t is None or t.numel() < n or t.dtype != dtype:
            t = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            self._bufs[name] = t
        return t[:n].view(*shape)

    def exchange_resources(self, world, experts):
        """Side stream, pinned host buffer and event for the count exchange (made once)."""
        r = getattr(self, "_exchange", None)
        if r is None:
            r = (torch.cuda.Stream(self.device),
                 torch.empty((world, experts), dtype=torch.int64).pin_memory(),
                 torch.cuda.Event())
            self._exchange = r
        return r

    def route(self, x):
        t, k, e = x.shape[0], self.cfg["top_k"], self.cfg["experts"]
        ids = self._buf("ids", (t, k), torch.int32)
        w = self._buf("w", (t, k), torch.float32)
        logits = self._buf("logits", (t, e), torch.float32)
        if not ops.k3_moe_route(self.layer.desc, ids, w, logits, x, t):
            raise RuntimeError("k3_moe_route failed")
        return ids, w

    def dispatch(self, ids, tokens, top_k, experts, tag):
        routes = tokens * top_k
        offsets = self._buf(tag + "off", (experts + 1,), torch.int32)
        sr = self._buf(tag + "sr", (routes,), torch.int32)
        st = self._buf(tag + "st", (routes,), torch.int32)
        inv = self._buf(tag + "inv", (routes,), torch.int32)
        nbytes = ops.k3_moe_dispatch_workspace_bytes(tokens, top_k, experts)
        ws = self._buf(tag + "ws", (nbytes,), torch.uint8)
        if not ops.k3_moe_dispatch_build(offsets, sr, st, inv, ids, tokens, top_k, experts, ws, nbytes):
            raise RuntimeError("k3_moe_dispatch_build failed")
        return offsets, sr, st, inv

    def gather(self, rows, index, tag):
        n, width = index.numel(), rows.shape[1]
        out = self._buf(tag, (n, width), rows.dtype)
        if n and not ops.k3_rocm_gather_rows_bf16(out, rows, index, n, width):
            raise RuntimeError("k3_rocm_gather_rows_bf16 failed")
        return out

    def experts(self, rows, offsets_local, index):
        """Expert products of rows[index] (grouped by local expert as offsets_local says)."""
        n, d, i = index.numel(), self.cfg["hidden"], self.cfg["expert_hidden"]
        out = self._buf("eo", (n, d), rows.dtype)
        act = self._buf("ea", (n, i), rows.dtype)
        if not n:
            return out
        # block-scaled path (gather folded into the row conversion) when the shape allows it
        need = ops.k3_moe_experts_workspace_bytes(self.layer.desc, n, rows.shape[0])
        if need:
            ws = self._buf("ews", (need,), torch.uint8)
            ok = ops.k3_moe_experts_grouped_ws(self.layer.desc, out, None, rows, index, rows.shape[0],
                                               offsets_local, n, ws, need)
        else:
            ok = ops.k3_moe_experts_grouped(self.layer.desc, out, act, self.gather(rows, index, "rows_in"),
                                            offsets_local, n)
        if not ok:
            raise RuntimeError("grouped expert products failed")
        return out

    def shared(self, x):
        s = self.cfg["shared_hidden"]
        if not s:
            return None
        t, d = x.shape
        out = self._buf("so", (t, d), x.dtype)
        g, u, a = (self._buf("s" + n, (t, s), x.dtype) for n in "gua")
        need = ops.k3_moe_shared_workspace_bytes(self.layer.desc, t)
        if need:
            ws = self._buf("sws", (need,), torch.uint8)
            ok = ops.k3_moe_shared_expert_ws(self.layer.desc, out, a, x, t, ws, need)
        else:
            ok = ops.k3_moe_shared_expert(self.layer.desc, out, g, u, a, x, t)
        if not ok:
            raise RuntimeError("k3_moe_shared_expert failed")
        return out

    def combine(self, rows, index, weights, shared, tokens):
        d, k = self.cfg["hidden"], self.cfg["top_k"]
        out = torch.empty((tokens, d), dtype=rows.dtype, device=self.device)
        if not ops.k3_moe_combine(out, rows, index, weights, shared, tokens, k, d):
            raise RuntimeError("k3_moe_combine failed")
        return out


def exchange_plan(all_counts: torch.Tensor, rank: int, first: int, per: int):
    """From the [world, E] matrix of rows each rank routes to each expert (host tensor):
    the all-to-all splits of this rank and, for the rows it receives (ordered source
    rank asc, expert asc, route asc), the gather index that regroups them (expert asc,
    source rank asc, route asc) with the local expert offsets [per + 1]."""
    world = all_counts.shape[0]
    own = all_counts[rank].reshape(world, -1).sum(dim=1)
    send = [int(v) for v in own]
    mine = all_counts[:, first:first + per]                        # [source, local expert]
    recv = [int(v) for v in mine.sum(dim=1)]
    src_base = torch.cumsum(mine.sum(dim=1), 0) - mine.sum(dim=1)  # first received row of each source
    within = torch.cumsum(mine, 1) - mine                          # offset of an expert inside a source's rows
    starts = (src_base[:, None] + within).t().reshape(-1)          # [expert, source] blocks of received rows
    lengths = mine.t().reshape(-1)
    offsets_local = torch.zeros(per + 1, dtype=torch.int64)
    offsets_local[1:] = torch.cumsum(mine.sum(dim=0), 0)
    return send, recv, starts, lengths, offsets_local


def rows_once_per_destination(world: int, top_k: int) -> bool:
    """Whether a pass sends each token row once per destination (plus a slot index per
    route) instead of once per route.  A token's top_k routes reach about
    world * (1 - (1 - 1/world)^top_k) distinct ranks; the bookkeeping pays when that
    cuts the rows at least threefold (16 routes: 2 and 4 ranks yes, 8 ranks no -
    measured 3.6 against 3.8 ms per pass there)."""
    distinct = world * (1.0 - (1.0 - 1.0 / world) ** top_k)
    return 3.0 * distinct <= top_k


def _ep_steps(backend, x, cfg: dict, group, once_per_destination=None):
    """One expert-parallel pass for the rows ``x`` as a generator: it yields after
    every point where the host has queued all it can without waiting, so that a
    driver can advance another pass (on another stream) in the meantime.  The
    value of the generator (StopIteration.value) is (out, ids, weights)."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    e, k = cfg["experts"], cfg["top_k"]
    first, per = shard_range(e, world, rank)
    t_local = x.shape[0]
    dev = x.device
    dedup = rows_once_per_destination(world, k) if once_per_destination is None else once_per_destination

    ids, weights = backend.route(x)
    offsets, sorted_route, sorted_token, inv_perm = backend.dispatch(ids, t_local, k, e, "src")

    # A token with several routes to one destination crosses the link once: per
    # destination g the source sends the rows of the tokens that have a route there
    # (token asc) and, per route, the slot of its token among them.
    # (Otherwise one row per route, in the sorted order, and no slots.)
    if dedup:
        dest = torch.div(ids.long(), per, rounding_mode="floor")                 # [T, k]
        member = torch.zeros((t_local, world), dtype=torch.int64, device=dev).scatter_(1, dest, 1)
        slots = torch.cumsum(member, 0) - 1                                       # [T, world]
        route_slot = slots[sorted_token.long(), dest.reshape(-1)[sorted_route.long()]].to(torch.int32)
        members_first = torch.argsort(member.t().reshape(-1), descending=True, stable=True)
        token_of_unique = (members_first % t_local).to(torch.int32)               # (destination asc, token asc)
        unique_counts = member.sum(0)
    else:
        token_of_unique = sorted_token
        unique_counts = torch.zeros(world, dtype=torch.int64, device=dev)

    # One collective and one host read tell every rank who sends how many rows of which
    # expert (and how many distinct token rows to whom).  On a GPU the exchange runs on
    # a side stream and the host reads it only after the shared expert has been queued,
    # so the device stays busy while the host waits and plans.
    counts = torch.cat([(offsets[1:] - offsets[:-1]).to(torch.int64), unique_counts])
    if x.is_cuda:
        main = torch.cuda.current_stream(dev)
        side, pinned, done = backend.exchange_resources(world, e + world)
        side.wait_stream(main)
        with torch.cuda.stream(side):
            counts.record_stream(side)
            gathered = [torch.empty_like(counts) for _ in range(world)]
            dist.all_gather(gathered, counts, group=group)
            pinned.copy_(torch.stack(gathered), non_blocking=True)
            done.record(side)
        shared = backend.shared(x)
        # every (destination, token) candidate row is gathered before the host knows how
        # many are members (members come first): the copy of the few surplus rows costs
        # less than leaving the device idle while the host plans
        rows_send = backend.gather(x, token_of_unique, "rows_send")
        yield
        done.synchronize()
        all_counts = pinned.clone()
    else:
        gathered = [torch.empty_like(counts) for _ in range(world)]
        dist.all_gather(gathered, counts, group=group)
        all_counts = torch.stack(gathered).cpu()
        shared = backend.shared(x)
        rows_send = backend.gather(x, token_of_unique, "rows_send")
        yield
    send, recv, starts, lengths, offsets_local = exchange_plan(all_counts[:, :e], rank, first, per)
    send_unique = [int(v) for v in all_counts[rank, e:]] if dedup else send
    recv_unique = [int(v) for v in all_counts[:, e + rank]] if dedup else recv
    n_recv, n_unique = sum(recv), sum(recv_unique)

    rows_send = rows_send[:sum(send_unique)]
    rows_recv = torch.empty((n_unique, x.shape[1]), dtype=x.dtype, device=dev)
    slots_arriving = None
    if dedup:
        slots_recv = torch.empty(n_recv, dtype=torch.int32, device=dev)
        slots_arriving = dist.all_to_all_single(slots_recv, route_slot, recv, send, group=group, async_op=True)
    arriving = dist.all_to_all_single(rows_recv.view(torch.uint8), rows_send.view(torch.uint8), recv_unique,
                                      send_unique, group=group, async_op=True)
    if n_recv:
        # gather index from the received order to the grouped order, built from the block
        # table while the rows are in flight
        # (one host-to-device copy for all the small tables)
        recv_unique_t = torch.tensor(recv_unique, dtype=torch.int64)
        tables = torch.cat([starts, lengths, offsets_local, torch.cumsum(recv_unique_t, 0) - recv_unique_t,
                            torch.tensor(recv, dtype=torch.int64)]).to(dev)
        n_blocks = starts.numel()
        starts_d, lengths_d = tables[:n_blocks], tables[n_blocks:2 * n_blocks]
        offsets_d = tables[2 * n_blocks:2 * n_blocks + per + 1].to(torch.int32)
        base_of_source, recv_d = tables[-2 * world:-world], tables[-world:]
        dest_base = torch.cumsum(lengths_d, 0) - lengths_d
        order = (torch.repeat_interleave(starts_d - dest_base, lengths_d, output_size=n_recv)
                 + torch.arange(n_recv, device=dev)).to(torch.int32)
        inverse = torch.empty_like(order)
        inverse[order.long()] = torch.arange(n_recv, device=dev, dtype=torch.int32)
        # first received row of each source, repeated for each of its routes
        if dedup:
            base_of_route = torch.repeat_interleave(base_of_source, recv_d, output_size=n_recv)
    yield
    if slots_arriving is not None:
        slots_arriving.wait()
    arriving.wait()
    if n_recv:
        # grouped position -> received route (-> row of its token among the received rows)
        row_of_route = (base_of_route + slots_recv.long())[order.long()].to(torch.int32) if dedup else order
        rows_out = backend.experts(rows_recv, offsets_d, row_of_route)
        rows_back = backend.gather(rows_out, inverse, "rows_back")   # received order again
    else:
        rows_back = torch.empty((0, x.shape[1]), dtype=x.dtype, device=dev)
    rows_home = torch.empty((t_local * k, x.shape[1]), dtype=x.dtype, device=dev)
    returning = dist.all_to_all_single(rows_home.view(torch.uint8), rows_back.view(torch.uint8), send, recv,
                                       group=group, async_op=True)
    yield
    returning.wait()
    return backend.combine(rows_home, inv_perm, weights, shared, t_local), ids, weights


def _drive(generators):
    """Advance the generators round-robin until all have returned; -> their values."""
    results = [None] * len(generators)
    live = list(range(len(generators)))
    while live:
        for i in list(live):
            try:
                next(generators[i])
            except StopIteration as stop:
                results[i] = stop.value
                live.remove(i)
    return results


def ep_forward(backend, x, cfg: dict, group=None, timings: dict | None = None, once_per_destination=None):
    """One expert-parallel layer pass for this rank's rows ``x`` [T_local, d]
    (2-byte elements: bf16, or int16 bit patterns on a CPU backend).
    ``once_per_destination`` forces the exchange form (default: ``rows_once_per_destination``)."""
    return _drive([_ep_steps(backend, x, cfg, group, once_per_destination)])[0]


def ep_forward_pipelined(backends, x, cfg: dict, group=None, streams=None):
    """The same pass with the rows cut into ``len(backends)`` consecutive pieces that
    advance in lock step, each with a backend (scratch buffers) of its own and, on
    a GPU, a stream of its own: while one piece's rows cross the links, another
    piece's kernels run.  Every rank must use the same number of pieces (the
    collectives pair up in issue order).  Rows are independent in every kernel of
    the pass, so the result equals ``ep_forward`` bit for bit."""
    pieces = len(backends)
    t = x.shape[0]
    bounds = [t * p // pieces for p in range(pieces + 1)]
    parts = [x[bounds[p]:bounds[p + 1]] for p in range(pieces)]
    if not x.is_cuda:
        results = _drive([_ep_steps(b, part, cfg, group) for b, part in zip(backends, parts)])
    else:
        main = torch.cuda.current_stream(x.device)

        def on_stream(gen, stream):
            # every step of a piece is issued with the piece's stream current
            while True:
                with torch.cuda.stream(stream):
                    try:
                        next(gen)
                    except StopIteration as stop:
                        return stop.value
                yield

        for s in streams:
            s.wait_stream(main)
        results = _drive([on_stream(_ep_steps(b, part, cfg, group), s)
                          for b, part, s in zip(backends, parts, streams)])
        for s, r in zip(streams, results):
            main.wait_stream(s)
            for tensor in r:
                tensor.record_stream(main)
        for s in streams:
            x.record_stream(s)
    out = torch.cat([r[0] for r in results])
    ids = torch.cat([r[1] for r in results])
    weights = torch.cat([r[2] for r in results])
    return out, ids, weights


def _bf16_ptr_ok(t: torch.Tensor) -> bool:
    return t.is_cuda and t.is_contiguous() and t.element_size() == 2


class ExpertParallelLayer:
    """The benchmark's layer sharded over the default process group (one rank per GPU).

    The pass itself is one call of ``k3_moe_ep_layer_forward``: the count exchange, both
    grouped send/recv steps and every kernel are issued by the library from C++ on the
    current stream.  ``torch.distributed`` is used once, to hand rank 0's NCCL identifier
    to the other ranks.  ``pieces`` > 1 selects the Python-driven pipelined form instead
    (``ep_forward_pipelined``; same results, kept for comparison)."""

    def __init__(self, cfg: dict, seed: int, device, tokens: int, weights: dict | None = None, pieces: int = 1,
                 reduced_return: bool = False):
        """``reduced_return``: the expert ranks return one weighted partial sum per (token, rank)
        instead of every expert row (``k3_moe_ep_set_reduced_return``): fewer bytes, results
        within the layer tolerance of the exact mode instead of bit-identical."""
        import ctypes as C
        self.world, self.rank = dist.get_world_size(), dist.get_rank()
        self.reduced_return = bool(reduced_return)
        if tokens % self.world != 0:
            raise ValueError("token count must divide evenly over the ranks")
        self.cfg = dict(cfg)
        self.tokens = tokens
        self.local_tokens = tokens // self.world
        first, per = shard_range(cfg["experts"], self.world, self.rank)
        self.layer = MoELayer(cfg, weights, seed=seed, device=device, local=(first, per), max_tokens=1)
        self.device = self.layer.device
        self.backends = [NativeBackend(self.layer) for _ in range(max(1, pieces))] if pieces > 1 else []
        self.streams = [torch.cuda.Stream(self.device) for _ in self.backends] if pieces > 1 else None
        # NCCL identifier from rank 0
        ident = torch.zeros(128, dtype=torch.uint8, device=self.device)
        err = C.create_string_buffer(256)
        if self.rank == 0:
            host = (C.c_uint8 * 128)()
            if not ops.k3_moe_ep_unique_id(C.addressof(host), err, 256):
                raise RuntimeError("k3_moe_ep_unique_id: " + err.value.decode())
            ident.copy_(torch.frombuffer(bytearray(host), dtype=torch.uint8))
        dist.broadcast(ident, 0)
        ident_host = (C.c_uint8 * 128).from_buffer_copy(ident.cpu().numpy().tobytes())
        handle = C.c_void_p()
        with torch.cuda.device(self.device):
            if not ops.k3_moe_ep_create(C.byref(handle), C.addressof(ident_host), self.rank, self.world, err, 256):
                raise RuntimeError("k3_moe_ep_create: " + err.value.decode())
        self.handle = handle
        if not ops.k3_moe_ep_set_reduced_return(self.handle, self.reduced_return):
            raise RuntimeError("k3_moe_ep_set_reduced_return failed")
        # every route of the batch may land on one rank: the sure bound
        self.max_recv = tokens * cfg["top_k"]
        need = ops.k3_moe_ep_workspace_bytes(self.handle, self.layer.desc, self.local_tokens, self.max_recv)
        if need == 0:
            raise RuntimeError("k3_moe_ep_workspace_bytes rejected the shard description")
        self.workspace = torch.empty(need, dtype=torch.uint8, device=self.device)
        self.decode_workspace = None

    def close(self):
        if getattr(self, "handle", None):
            torch.cuda.synchronize(self.device)
            ops.k3_moe_ep_destroy(self.handle)
            self.handle = None

    def forward(self, x: torch.Tensor, want_routes: bool = False):
        import ctypes as C
        if self.backends:
            out, ids, w = ep_forward_pipelined(self.backends, x, self.cfg, streams=self.streams)
            return (out, ids, w) if want_routes else out
        t, k = x.shape[0], self.cfg["top_k"]
        assert t <= self.local_tokens and _bf16_ptr_ok(x)
        out = torch.empty_like(x)
        ids = torch.empty((t, k), dtype=torch.int32, device=self.device) if want_routes else None
        w = torch.empty((t, k), dtype=torch.float32, device=self.device) if want_routes else None
        err = C.create_string_buffer(256)
        if not ops.k3_moe_ep_layer_forward(self.handle, self.layer.desc, out, x, t, self.max_recv, self.workspace,
                                           self.workspace.numel(), ids, w, err, 256):
            raise RuntimeError("k3_moe_ep_layer_forward: " + err.value.decode())
        return (out, ids, w) if want_routes else out

    def decode(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        """One token, the same on every rank: x bf16 [1, d] -> out bf16 [1, d] on every rank."""
        if self.decode_workspace is None:
            need = ops.k3_moe_ep_decode_workspace_bytes(self.handle, self.layer.desc)
            if need == 0:
                raise RuntimeError("the one-token path does not take this layer shape")
            self.decode_workspace = torch.empty(need, dtype=torch.uint8, device=self.device)
        out = torch.empty_like(x)
        if not ops.k3_moe_ep_decode(self.handle, self.layer.desc, out, x, residual, self.decode_workspace,
                                    self.decode_workspace.numel()):
            raise RuntimeError("k3_moe_ep_decode failed")
        return out

    def phase_times(self, x: torch.Tensor, steps: int = 5) -> dict:
        """Device time of the grouped expert products on this rank's received rows and of
        the whole pass, averaged over ``steps`` passes (events recorded by the library)."""
        import ctypes as C
        experts = total = 0.0
        rows = 0
        e, p, n = C.c_float(), C.c_float(), C.c_uint32()
        for _ in range(steps):
            self.forward(x)
            if not ops.k3_moe_ep_last_pass(self.handle, C.byref(e), C.byref(p), C.byref(n)):
                raise RuntimeError("k3_moe_ep_last_pass failed")
            experts += e.value
            total += p.value
            rows = n.value
        return {"experts_ms": experts / steps, "pass_ms": total / steps, "recv_rows": rows}


class DecodeStack:
    """A stack of routed-MoE layers decoding one token at a time, expert-parallel over
    the default process group (or on one GPU without one): ``layers`` layer positions
    backed by ``distinct`` resident weight sets used round-robin (position l uses set
    l % distinct).  One call of ``k3_moe_ep_decode_stack`` per token."""

    def __init__(self, cfg: dict, layers: int, distinct: int, device, seed: int = 0):
        import ctypes as C
        from . import _native
        if dist.is_available() and dist.is_initialized():
            self.world, self.rank = dist.get_world_size(), dist.get_rank()
        else:
            self.world, self.rank = 1, 0
        self.cfg, self.layers, self.distinct = dict(cfg), layers, min(distinct, layers)
        self.device = torch.device(device)
        first, per = shard_range(cfg["experts"], self.world, self.rank)
        self.sets = [MoELayer(cfg, None, seed=seed + i, device=device, local=(first, per), max_tokens=1)
                     for i in range(self.distinct)]
        err = C.create_string_buffer(256)
        handle = C.c_void_p()
        ident_host = None
        if self.world > 1:
            ident = torch.zeros(128, dtype=torch.uint8, device=self.device)
            if self.rank == 0:
                host = (C.c_uint8 * 128)()
                if not ops.k3_moe_ep_unique_id(C.addressof(host), err, 256):
                    raise RuntimeError("k3_moe_ep_unique_id: " + err.value.decode())
                ident.copy_(torch.frombuffer(bytearray(host), dtype=torch.uint8))
            dist.broadcast(ident, 0)
            ident_host = (C.c_uint8 * 128).from_buffer_copy(ident.cpu().numpy().tobytes())
        with torch.cuda.device(self.device):
            if not ops.k3_moe_ep_create(C.byref(handle), C.addressof(ident_host) if ident_host else None,
                                        self.rank, self.world, err, 256):
                raise RuntimeError("k3_moe_ep_create: " + err.value.decode())
        self.handle = handle
        self.table = (C.POINTER(_native.LayerDesc) * layers)(
            *[C.pointer(self.sets[l % self.distinct].desc) for l in range(layers)])
        need = ops.k3_moe_ep_decode_workspace_bytes(self.handle, self.sets[0].desc)
        if need == 0:
            raise RuntimeError("the one-token path does not take this layer shape")
        d = cfg["hidden"]
        self.workspace = torch.empty(need + 3 * (2 * d + 256) + 1024, dtype=torch.uint8, device=self.device)
        self.norm_weight = torch.ones(d, dtype=torch.bfloat16, device=self.device)

    def step(self, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        out = torch.empty_like(x) if out is None else out
        if not ops.k3_moe_ep_decode_stack(self.handle, self.table, self.layers, out, x, self.norm_weight, 1e-5,
                                          self.workspace, self.workspace.numel()):
            raise RuntimeError("k3_moe_ep_decode_stack failed")
        return out

    def weight_bytes(self) -> int:
        return sum(s.weight_bytes() for s in self.sets)

    def close(self):
        if getattr(self, "handle", None):
            torch.cuda.synchronize(self.device)
            ops.k3_moe_ep_destroy(self.handle)
            self.handle = None
