"""Worker of tests/test_gpu_ep.py: one rank per GPU (launched by torch.distributed.run).
Compares the expert-parallel layer with the single-GPU layer on the same seeded
inputs and writes an outcome line per rank."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from moonshine_b200 import synth                                   # noqa: E402
from moonshine_b200.ep import ExpertParallelLayer                  # noqa: E402
from moonshine_b200.layer import MoELayer, bf16_tensor_to_bits     # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    outcomes = []
    # at least 32 local tokens per rank: fewer take the matrix-vector kernels for the router and the
    # shared expert, which differ from the single-GPU layer's tensor-core kernels in the last bits
    for bias_mode, tokens in (("uniform", max(128, 32 * world)), ("hot4", max(256, 32 * world))):
        cfg = synth.baseline_config(hidden=1024, expert_hidden=512, experts=64, top_k=8,
                                    shared_hidden=512, bias_mode=bias_mode)
        weights = synth.make_layer(cfg, seed=5)
        x = synth.activations(5, tokens, cfg["hidden"])
        per = tokens // world
        xl = torch.from_numpy(x[rank * per:(rank + 1) * per].view(np.int16).copy()).to(device).view(torch.bfloat16)
        ep_layer = ExpertParallelLayer(cfg, seed=5, device=device, tokens=tokens, weights=weights)
        out, ids, w = ep_layer.forward(xl, want_routes=True)
        single = MoELayer(cfg, weights, seed=5, device=device, max_tokens=tokens)
        xs = torch.from_numpy(x.view(np.int16).copy()).to(device).view(torch.bfloat16)
        ref, ref_ids, ref_w = single.forward(xs, want_routes=True)
        torch.cuda.synchronize()
        got, want = bf16_tensor_to_bits(out), bf16_tensor_to_bits(ref)[rank * per:(rank + 1) * per]
        same_ids = bool(torch.equal(ids, ref_ids[rank * per:(rank + 1) * per]))
        g = (got.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        r = (want.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        rel = float(np.sqrt(((g - r) ** 2).sum() / (r ** 2).sum()))
        outcomes.append((bias_mode, same_ids, bool(np.array_equal(got, want)), rel))
        # both forms of the exchange (a row per route / a row per destination): same bits
        from moonshine_b200.ep import NativeBackend, ep_forward
        python_path = NativeBackend(ep_layer.layer)      # the same pass driven from Python
        for form in (False, True):
            out1, ids1, _ = ep_forward(python_path, xl, cfg, once_per_destination=form)
            torch.cuda.synchronize()
            same = bool(np.array_equal(bf16_tensor_to_bits(out1), got)) and bool(torch.equal(ids1, ids))
            outcomes.append((bias_mode + ("/row per destination" if form else "/row per route"), same, same,
                             0.0 if same else 1.0))
        # the same pass cut into two row ranges pipelined against each other: same bits, as long
        # as every range still has enough rows for the same kernels (>= 32 routed rows per rank)
        if per // 2 * cfg["top_k"] // world >= 64:
            piped = ExpertParallelLayer(cfg, seed=5, device=device, tokens=tokens, weights=weights, pieces=2)
            for _ in range(3):
                out2, ids2, _ = piped.forward(xl, want_routes=True)
            torch.cuda.synchronize()
            same = bool(np.array_equal(bf16_tensor_to_bits(out2), got)) and bool(torch.equal(ids2, ids))
            outcomes.append((bias_mode + "/pipelined", same, same, 0.0 if same else 1.0))
            piped.close()
        # reduced return (one partial sum per token and expert rank): same routing, output within
        # the layer tolerance of the exact result
        reduced = ExpertParallelLayer(cfg, seed=5, device=device, tokens=tokens, weights=weights, reduced_return=True)
        for _ in range(2):
            out3, ids3, _ = reduced.forward(xl, want_routes=True)
        torch.cuda.synchronize()
        g3 = (bf16_tensor_to_bits(out3).astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        rel3 = float(np.sqrt(((g3 - r) ** 2).sum() / (r ** 2).sum()))
        outcomes.append((bias_mode + "/reduced return", bool(torch.equal(ids3, ids)), rel3 <= 1e-2, min(rel3, 1e-3)))
        sys.stderr.write(f"rank {rank}: reduced return rel-L2 {rel3:.2e}\n")
        reduced.close()
        # one token, replicated: every rank must end with the single-GPU layer's row
        for t in (0, 3):
            one = ep_layer.decode(xs[t:t + 1])
            want_one = single.forward(xs[t:t + 1])
            torch.cuda.synchronize()
            same = bool(torch.equal(one, want_one))
            outcomes.append((f"{bias_mode}/one token {t}", same, same, 0.0 if same else 1.0))
        ep_layer.close()
    # a stack of 6 layer positions over 3 weight sets, one token at a time, against the
    # same stack on one GPU (a handle of world size 1 in this process)
    from moonshine_b200.ep import DecodeStack
    cfg = synth.baseline_config(hidden=1024, expert_hidden=512, experts=64, top_k=8, shared_hidden=512)
    stack = DecodeStack(cfg, layers=6, distinct=3, device=device, seed=40)
    x0 = torch.from_numpy(synth.activations(41, 2, cfg["hidden"]).view(np.int16).copy()).to(device).view(torch.bfloat16)
    got_stack = [stack.step(x0[t:t + 1]).clone() for t in range(2)]
    torch.cuda.synchronize()
    stack.close()
    h = [x0[t:t + 1].clone() for t in range(2)]
    import ctypes as C
    from moonshine_b200 import ops
    norm_w = torch.ones(cfg["hidden"], dtype=torch.bfloat16, device=device)
    for l in range(6):
        full = MoELayer(cfg, None, seed=40 + l % 3, device=device, max_tokens=1)
        ws_bytes = ops.k3_moe_block_workspace_bytes(full.desc, 1)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=device)
        for t in range(2):
            nxt = torch.empty_like(h[t])
            assert ops.k3_moe_block_forward(full.desc, nxt, h[t], norm_w, 1e-5, 1, ws, ws_bytes)
            h[t] = nxt
        torch.cuda.synchronize()
        del full, ws
    for t in range(2):
        same = bool(torch.equal(got_stack[t], h[t]))
        outcomes.append((f"stack token {t}", same, same, 0.0 if same else 1.0))
    ok = all(v[1] and v[2] and v[3] <= 1e-3 for v in outcomes)
    sys.stderr.write(f"rank {rank}: {outcomes}\n")
    # one outcome line for the whole job (lines of several ranks could interleave)
    flag = torch.tensor([1 if ok else 0], device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    all_ok = bool(flag.item())
    if rank == 0:
        print(f"EP_RESULT ranks={world} ok={all_ok}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if all_ok else 1)


if __name__ == "__main__":
    main()
