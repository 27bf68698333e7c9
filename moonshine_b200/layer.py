"""Slot table and fused layer on one GPU (host-side mirror of the MoE half of the
reference's ``decode_routed_layer`` / ``prefill_routed_layer``).

``MoELayer`` owns the device tensors of one layer (router, expert slot table,
shared expert), the ``k3_moe_layer_desc`` describing them and a workspace sized
for a maximum token count.  ``forward`` is one call of ``k3_moe_layer_forward``.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _native, ops, synth


def _dev(a: np.ndarray, device) -> torch.Tensor:
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:                       # bf16 bit patterns
        return torch.from_numpy(a.view(np.int16)).to(device).view(torch.bfloat16)
    if a.dtype == np.uint32:
        return torch.from_numpy(a.view(np.int32)).to(device)
    return torch.from_numpy(a).to(device)


def bf16_tensor_to_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


class MoELayer:
    """One routed-MoE layer resident in HBM.

    ``cfg`` is a config dict as produced by ``synth.baseline_config``.  Expert
    tensors are either uploaded from ``weights`` (numpy, small shapes) or filled
    on the device from the same seeded streams (``weights`` without expert
    entries), which is bit-identical.  ``local`` = (first, count) selects the
    expert-parallel shard held by this GPU (default: all experts).
    """

    def __init__(self, cfg: dict, weights: dict | None = None, seed: int = 0,
                 device="cuda:0", local: tuple[int, int] | None = None, max_tokens: int = 1):
        self.cfg = dict(cfg)
        self.device = torch.device(device)
        self.seed = seed
        d, i, e, s = cfg["hidden"], cfg["expert_hidden"], cfg["experts"], cfg["shared_hidden"]
        first, count = local if local is not None else (0, e)
        self.local_first, self.local_count = first, count
        if weights is None:
            weights = synth.make_layer(cfg, seed, experts=False)
        self.t = {}
        self.t["router_weight"] = _dev(weights["router_weight"], self.device)
        self.t["router_bias"] = _dev(weights["router_bias"], self.device)
        with torch.cuda.device(self.device):
            for name, (tp, ts, rows, cols) in synth.expert_tensor_specs(cfg).items():
                for suffix, tag, per in (("_packed", tp, rows * cols // 2), ("_scales", ts, rows * cols // 32)):
                    key = name + suffix
                    if key in weights:
                        self.t[key] = _dev(weights[key][first:first + count], self.device)
                    else:
                        buf = torch.empty(count * per, dtype=torch.uint8, device=self.device)
                        self._fill_expert_bytes(buf, tag, per, suffix == "_scales")
                        self.t[key] = buf
            if s:
                for name in synth.shared_tensor_specs(cfg):
                    self.t[name + "_q"] = _dev(weights[name + "_q"], self.device)
                    self.t[name + "_s"] = _dev(weights[name + "_s"], self.device)
        self.desc = _native.LayerDesc(
            hidden=d, expert_hidden=i, expert_count=e, top_k=cfg["top_k"], shared_hidden=s,
            q8_block=cfg["q8_block"], q8_scale_type=cfg["q8_scale_type"],
            activation=cfg["activation"], beta=cfg["beta"], linear_beta=cfg["linear_beta"],
            route_scale=cfg["route_scale"], local_expert_first=first, local_expert_count=count,
            router_weight=self.t["router_weight"].data_ptr(),
            router_bias=self.t["router_bias"].data_ptr(),
            w1_packed=self.t["w1_packed"].data_ptr(), w1_scales=self.t["w1_scales"].data_ptr(),
            w3_packed=self.t["w3_packed"].data_ptr(), w3_scales=self.t["w3_scales"].data_ptr(),
            w2_packed=self.t["w2_packed"].data_ptr(), w2_scales=self.t["w2_scales"].data_ptr(),
            shared_gate_q=self.t["shared_gate_q"].data_ptr() if s else None,
            shared_gate_s=self.t["shared_gate_s"].data_ptr() if s else None,
            shared_up_q=self.t["shared_up_q"].data_ptr() if s else None,
            shared_up_s=self.t["shared_up_s"].data_ptr() if s else None,
            shared_down_q=self.t["shared_down_q"].data_ptr() if s else None,
            shared_down_s=self.t["shared_down_s"].data_ptr() if s else None,
        )
        self.max_tokens = 0
        self.workspace = None
        self.reserve(max_tokens)

    # ------------------------------------------------------------------ setup
    def _fill_expert_bytes(self, buf, tag, per_expert, is_scale):
        """Fill the shard [first, first+count) of a per-expert byte tensor from the
        seeded stream of the *whole* layer, so shards equal slices of the full tensor."""
        cfg = self.cfg
        key = synth.stream_key(self.seed, tag)
        start = self.local_first * per_expert
        if start % 8 != 0:
            raise ValueError("expert tensor size must be a multiple of 8 bytes")
        low, span = (cfg["scale_low"], cfg["scale_span"]) if is_scale else (0, 256)
        if not ops.k3_synth_fill_bytes(buf, buf.numel(), key, start, low, span):
            raise RuntimeError("k3_synth_fill_bytes failed")

    def reserve(self, max_tokens: int) -> None:
        if max_tokens <= self.max_tokens:
            return
        need = ops.k3_moe_layer_workspace_bytes(self.desc, max_tokens)
        if need == 0:
            raise RuntimeError("k3_moe_layer_workspace_bytes rejected the layer description")
        self.workspace = torch.empty(need, dtype=torch.uint8, device=self.device)
        self.max_tokens = max_tokens

    # ---------------------------------------------------------------- forward
    def forward(self, x: torch.Tensor, want_routes: bool = False):
        """x bf16 [tokens, d] on this device -> out bf16 [tokens, d]
        (and ids int32 / weights f32 [tokens, top_k] when ``want_routes``)."""
        tokens = x.shape[0]
        self.reserve(tokens)
        out = torch.empty_like(x)
        ids = wts = None
        if want_routes:
            ids = torch.empty((tokens, self.cfg["top_k"]), dtype=torch.int32, device=self.device)
            wts = torch.empty((tokens, self.cfg["top_k"]), dtype=torch.float32, device=self.device)
        ok = ops.k3_moe_layer_forward(self.desc, out, x, tokens, self.workspace,
                                      self.workspace.numel(), ids, wts)
        if not ok:
            raise RuntimeError("k3_moe_layer_forward failed")
        return (out, ids, wts) if want_routes else out

    def phase_times(self, x: torch.Tensor, steps: int = 5) -> dict:
        """Average device time of each phase over ``steps`` passes, from CUDA events
        recorded by the library on the launching stream."""
        tokens = x.shape[0]
        self.reserve(tokens)
        out = torch.empty_like(x)
        names = ["router_ms", "shared_ms", "dispatch_ms", "experts_ms", "combine_ms"]
        total = dict.fromkeys(names, 0.0)
        events = [ops.k3_moe_event_create() for _ in range(6)]
        if not all(events):
            raise RuntimeError("cudaEventCreate failed")
        arr = (C.c_void_p * 6)(*events)
        try:
            for _ in range(steps):
                if not ops.k3_moe_layer_forward_events(self.desc, out, x, tokens, self.workspace,
                                                       self.workspace.numel(), arr):
                    raise RuntimeError("k3_moe_layer_forward_events failed")
                for i, name in enumerate(names):
                    total[name] += ops.k3_moe_event_elapsed_ms(events[i], events[i + 1])
        finally:
            for e in events:
                ops.k3_moe_event_destroy(e)
        return {k: v / steps for k, v in total.items()}

    def weight_bytes(self) -> int:
        return sum(v.numel() * v.element_size() for v in self.t.values())


class LatentMoELayer:
    """The routed layer at the model's real shape: router and shared expert at the
    model width ``cfg['hidden']``, experts on a latent projection of width
    ``latent`` (``k3_moe_latent_layer_forward``).  Tensors are seeded synthetic."""

    def __init__(self, cfg: dict, latent: int, seed: int = 0, device="cuda:0", max_tokens: int = 1,
                 norm_epsilon: float = 1e-5):
        self.cfg = dict(cfg)
        self.latent = latent
        self.device = torch.device(device)
        h = cfg["hidden"]
        # expert tables at the latent width (a MoELayer without shared expert owns them),
        # router and shared expert at the model width
        inner_cfg = dict(cfg, hidden=latent, shared_hidden=0)
        self.inner = MoELayer(inner_cfg, None, seed=seed + 1, device=device, max_tokens=1)
        outer = synth.make_layer(cfg, seed, experts=False)
        self.t = {k: _dev(v, self.device) for k, v in outer.items() if k != "config"}
        blk = cfg["q8_block"]
        sdt = torch.float16 if cfg["q8_scale_type"] == synth.Q8_F16 else torch.float32
        with torch.cuda.device(self.device):
            for name, rows, cols, tag in (("down", latent, h, 911), ("up", h, latent, 913)):
                q = torch.empty((rows, cols), dtype=torch.int8, device=self.device)
                sc = torch.empty((rows, cols // blk), dtype=sdt, device=self.device)
                if not ops.k3_synth_fill_int8(q, q.numel(), synth.stream_key(seed, tag), 0) or \
                        not ops.k3_synth_fill_uniform(sc, sc.numel(), synth.stream_key(seed, tag + 1), 0,
                                                      1e-4, 9e-4, 1 if sdt is torch.float16 else 0):
                    raise RuntimeError("synthetic fill failed")
                self.t[name + "_q"], self.t[name + "_s"] = q, sc
            self.t["norm_w"] = torch.ones(latent, dtype=torch.bfloat16, device=self.device)
        self.desc = _native.LatentDesc()
        C.memmove(C.byref(self.desc.layer), C.byref(self.inner.desc), C.sizeof(_native.LayerDesc))
        lay = self.desc.layer
        lay.hidden, lay.shared_hidden = h, cfg["shared_hidden"]
        for name in ("router_weight", "router_bias"):
            setattr(lay, name, self.t[name].data_ptr())
        if cfg["shared_hidden"]:
            for name in synth.shared_tensor_specs(cfg):
                setattr(lay, name + "_q", self.t[name + "_q"].data_ptr())
                setattr(lay, name + "_s", self.t[name + "_s"].data_ptr())
        self.desc.latent, self.desc.norm_epsilon = latent, norm_epsilon
        self.desc.down_q, self.desc.down_s = self.t["down_q"].data_ptr(), self.t["down_s"].data_ptr()
        self.desc.up_q, self.desc.up_s = self.t["up_q"].data_ptr(), self.t["up_s"].data_ptr()
        self.desc.norm_weight = self.t["norm_w"].data_ptr()
        self.max_tokens = 0
        self.workspace = None
        self.reserve(max_tokens)

    def reserve(self, max_tokens: int) -> None:
        if max_tokens <= self.max_tokens:
            return
        need = ops.k3_moe_latent_workspace_bytes(self.desc, max_tokens)
        if need == 0:
            raise RuntimeError("k3_moe_latent_workspace_bytes rejected the layer description")
        self.workspace = torch.empty(need, dtype=torch.uint8, device=self.device)
        self.max_tokens = max_tokens

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        tokens = x.shape[0]
        self.reserve(tokens)
        out = torch.empty_like(x)
        if not ops.k3_moe_latent_layer_forward(self.desc, out, x, tokens, self.workspace,
                                               self.workspace.numel(), None, None):
            raise RuntimeError("k3_moe_latent_layer_forward failed")
        return out
