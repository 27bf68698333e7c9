"""Partially resident expert store: expert weights stay in host memory as
checkpoint spans, a fixed number of device slots per layer holds the experts in
use, and the slot policy is the reference's token-batch LRU with its plan /
commit hand-over (k3_expert_cache.h:44-53, planned at k3_engine.cu:1600-1612 and
committed at :1904).

``SlotCache`` binds the policy (host code in the native library,
include/k3_moe_store.h).  ``PartialStore`` runs one token's routed experts out of
the slots: plan -> admit the misses into their destination slots
(``k3_moe_store_admit``, stream-ordered behind the readers of the previous token)
-> expert products addressed by slot -> weighted sum -> commit.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _native

SPAN_ORDER = ("w1_packed", "w1_scales", "w2_packed", "w2_scales", "w3_packed", "w3_scales")


class StoreError(RuntimeError):
    """A slot-policy call returned false; the message is the library's."""


def span_layout(hidden: int, expert_hidden: int) -> tuple[list[int], int]:
    """Relative byte offsets of the six tensors of one expert's checkpoint span
    (w1.packed, w1.scale, w2.packed, w2.scale, w3.packed, w3.scale, stored back
    to back: k3_engine.cu:951-1030) and the span's size.  At the reference's
    shape (3584 x 3072) this gives 0 / 5,505,024 / 5,849,088 / 11,354,112 /
    11,698,176 / 17,203,200 and 17,547,264 bytes."""
    up = expert_hidden * hidden          # elements of w1 / w3 [I, d]
    down = hidden * expert_hidden        # elements of w2 [d, I]
    sizes = [up // 2, up // 32, down // 2, down // 32, up // 2, up // 32]
    offsets = [0]
    for s in sizes[:-1]:
        offsets.append(offsets[-1] + s)
    return offsets, offsets[-1] + sizes[-1]


def pack_spans(weights: dict, experts: int, hidden: int, expert_hidden: int) -> np.ndarray:
    """Per-expert tensors (numpy, [E, ...]) -> spans u8 [E, span_bytes] in checkpoint order."""
    offsets, total = span_layout(hidden, expert_hidden)
    spans = np.empty((experts, total), dtype=np.uint8)
    for name, off in zip(SPAN_ORDER, offsets):
        flat = np.ascontiguousarray(weights[name]).reshape(experts, -1).view(np.uint8)
        spans[:, off:off + flat.shape[1]] = flat
    return spans


class SlotCache:
    """The slot policy.  ``prefix`` / ``handle`` let the same wrapper drive another
    build of the same interface (the tests point it at the reference's own C file
    compiled as a checker)."""

    def __init__(self, layers: int, slots_per_layer: int, handle=None, prefix: str = "k3_moe_slot_cache_"):
        self._lib = handle if handle is not None else _native.lib()
        self._prefix = prefix
        self.layers, self.slots_per_layer = layers, slots_per_layer
        self._err = C.create_string_buffer(256)
        self._cache = C.c_void_p()
        if handle is not None:
            self._declare()
        if not self._fn("create")(C.byref(self._cache), layers, slots_per_layer, self._err, len(self._err)):
            raise StoreError(self._err.value.decode())

    def _declare(self):
        for name, (restype, argtypes) in _native.SIGNATURES.items():
            if name.startswith("k3_moe_slot_cache_") and name != "k3_moe_slot_cache_replay_line":
                fn = getattr(self._lib, self._prefix + name[len("k3_moe_slot_cache_"):])
                fn.restype, fn.argtypes = restype, argtypes

    def _fn(self, name):
        return getattr(self._lib, self._prefix + name)

    def _check(self, ok):
        if not ok:
            raise StoreError(self._err.value.decode())

    def close(self):
        if self._cache:
            self._fn("destroy")(self._cache)
            self._cache = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def plan(self, layer: int, expert_ids) -> list[tuple[bool, bool, int, int]]:
        """-> per rank (hit, admit, source_slot, destination_slot); slots are global."""
        n = len(expert_ids)
        ids = (C.c_uint16 * max(n, 1))(*[int(e) for e in expert_ids])
        acc = (_native.SlotAccess * max(n, 1))()
        self._check(self._fn("plan")(self._cache, layer, ids if n else None, n, acc, self._err, len(self._err)))
        return [(bool(a.hit), bool(a.admit), int(a.source_slot), int(a.destination_slot)) for a in acc[:n]]

    def commit(self, layer: int) -> None:
        self._check(self._fn("commit")(self._cache, layer, self._err, len(self._err)))

    def abort(self, layer: int) -> None:
        self._fn("abort")(self._cache, layer)

    def stats(self) -> dict:
        st = _native.SlotStats()
        self._fn("get_stats")(self._cache, C.byref(st))
        return {name: int(getattr(st, name)) for name, _ in _native.SlotStats._fields_}

    def snapshot(self, layer: int) -> list[int]:
        ids = (C.c_uint16 * self.slots_per_layer)()
        count = C.c_uint16()
        self._check(self._fn("snapshot_layer")(self._cache, layer, ids, self.slots_per_layer, C.byref(count),
                                              self._err, len(self._err)))
        return [int(v) for v in ids[:count.value]]

    def reset(self) -> None:
        self._check(self._fn("reset")(self._cache, self._err, len(self._err)))

    def invalidate_slots(self, first_slot: int, slot_count: int) -> None:
        self._check(self._fn("invalidate_slots")(self._cache, first_slot, slot_count, self._err, len(self._err)))

    def slot_count(self) -> int:
        return int(self._fn("slot_count")(self._cache))

    def storage_bytes(self, bytes_per_expert: int) -> int:
        return int(self._fn("storage_bytes")(self._cache, bytes_per_expert))

    def replay_line(self, layer: int, expert_ids) -> tuple[int, int]:
        """plan + commit of one trace line -> (hit mask, admissions)."""
        n = len(expert_ids)
        ids = (C.c_uint16 * max(n, 1))(*[int(e) for e in expert_ids])
        mask, admitted = C.c_uint32(), C.c_uint32()
        self._check(self._fn("replay_line")(self._cache, layer, ids, n, C.byref(mask), C.byref(admitted),
                                           self._err, len(self._err)))
        return int(mask.value), int(admitted.value)


class PartialStore:
    """One layer's routed experts served from ``slots`` device slots.

    ``spans`` is a pinned host tensor u8 [experts, span_bytes] in checkpoint order
    (``pack_spans``).  ``cache``/``layer`` may be shared between the stores of
    several layers; by default the store owns a one-layer cache.
    """

    def __init__(self, cfg: dict, spans, slots: int, device="cuda:0", cache: SlotCache | None = None,
                 layer: int = 0):
        import torch
        from . import ops
        self._torch, self._ops = torch, ops
        self.cfg = dict(cfg)
        self.device = torch.device(device)
        d, i, k = cfg["hidden"], cfg["expert_hidden"], cfg["top_k"]
        if slots < k:
            raise ValueError("a layer needs at least top_k slots: every expert of a token is resident while it runs")
        self.slots, self.layer = slots, layer
        self.cache = cache if cache is not None else SlotCache(1, slots)
        self.spans = spans
        self.relative, self.span_bytes = span_layout(d, i)
        if spans.shape[1] != self.span_bytes:
            raise ValueError("span size does not match the layer shape")
        self._relative = (C.c_uint64 * 6)(*self.relative)
        sizes = {"w1_packed": i * d // 2, "w1_scales": i * d // 32, "w2_packed": d * i // 2,
                 "w2_scales": d * i // 32, "w3_packed": i * d // 2, "w3_scales": i * d // 32}
        self.t = {name: torch.zeros(slots * n, dtype=torch.uint8, device=self.device) for name, n in sizes.items()}
        self.desc = _native.LayerDesc(
            hidden=d, expert_hidden=i, expert_count=slots, top_k=k, shared_hidden=0,
            q8_block=cfg["q8_block"], q8_scale_type=cfg["q8_scale_type"], activation=cfg["activation"],
            beta=cfg["beta"], linear_beta=cfg["linear_beta"], route_scale=cfg["route_scale"],
            local_expert_first=0, local_expert_count=slots,
            **{name: self.t[name].data_ptr() for name in sizes})
        u32 = dict(dtype=torch.int32, device=self.device)
        self.slot_ids = torch.empty((1, k), **u32)
        self.slot_ids_host = torch.empty((1, k), dtype=torch.int32).pin_memory()
        self.offsets = torch.empty(slots + 1, **u32)
        self.sorted_route, self.sorted_token, self.inv_perm = (torch.empty(k, **u32) for _ in range(3))
        self.dispatch_ws = torch.empty(max(1, ops.k3_moe_dispatch_workspace_bytes(1, k, slots)), dtype=torch.uint8,
                                       device=self.device)
        self.rows_in = torch.empty((k, d), dtype=torch.bfloat16, device=self.device)
        self.act = torch.empty((k, i), dtype=torch.bfloat16, device=self.device)
        self.rows_out = torch.empty((k, d), dtype=torch.bfloat16, device=self.device)
        # the one-token expert kernel takes slot numbers as expert ids (shapes it handles)
        token_bytes = ops.k3_moe_experts_token_workspace_bytes(self.desc)
        self.token_ws = (torch.empty(token_bytes, dtype=torch.uint8, device=self.device) if token_bytes else None)
        self.bytes_admitted = 0

    def token(self, x, expert_ids, weights):
        """x bf16 [1, d] and weights f32 [top_k] on the device, expert_ids on the
        host (the reference plans from host copies too, k3_engine.cu:1580-1590) ->
        (weighted sum bf16 [1, d], hit mask)."""
        torch, ops = self._torch, self._ops
        k, d = self.cfg["top_k"], self.cfg["hidden"]
        accesses = self.cache.plan(self.layer, expert_ids)
        try:
            mask = 0
            for rank, (hit, admit, source, destination) in enumerate(accesses):
                if hit:
                    mask |= 1 << rank
                    slot = source
                elif admit:
                    slot = destination
                    # same stream as the expert kernels: the copy lands after the readers
                    # of the slot's previous content have finished
                    if not ops.k3_moe_store_admit(self.desc, slot - self.layer * self.slots,
                                                  self.spans[int(expert_ids[rank])].data_ptr(), self._relative):
                        raise StoreError("k3_moe_store_admit failed")
                    self.bytes_admitted += self.span_bytes
                else:
                    raise StoreError("expert neither resident nor admitted: fewer slots than experts per token")
                self.slot_ids_host[0, rank] = slot - self.layer * self.slots
            self.slot_ids.copy_(self.slot_ids_host, non_blocking=True)
            out = torch.empty((1, d), dtype=torch.bfloat16, device=self.device)
            if self.token_ws is not None:
                # the block-scaled one-token expert kernel, addressed by slot number
                ok = ops.k3_moe_experts_token(self.desc, out, x, self.slot_ids, weights, self.token_ws,
                                              self.token_ws.numel())
            else:
                ok = ops.k3_moe_dispatch_build(self.offsets, self.sorted_route, self.sorted_token, self.inv_perm,
                                               self.slot_ids, 1, k, self.slots, self.dispatch_ws,
                                               self.dispatch_ws.numel())
                ok = ok and ops.k3_rocm_gather_rows_bf16(self.rows_in, x, self.sorted_token, k, d)
                ok = ok and ops.k3_moe_experts_grouped(self.desc, self.rows_out, self.act, self.rows_in, self.offsets, k)
                ok = ok and ops.k3_moe_combine(out, self.rows_out, self.inv_perm, weights, None, 1, k, d)
            if not ok:
                raise StoreError("expert products failed")
            # the pinned id buffer is rewritten by the next token
            torch.cuda.current_stream(self.device).synchronize()
        except Exception:
            self.cache.abort(self.layer)
            raise
        self.cache.commit(self.layer)
        return out, mask
