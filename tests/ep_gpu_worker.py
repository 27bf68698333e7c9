"""Worker of tests/test_gpu_ep.py: one rank per GPU (launched by torch.distributed.run).
Compares the expert-parallel layer with the single-GPU layer on the same seeded
inputs and writes a verdict line per rank."""
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
    verdicts = []
    for bias_mode, tokens in (("uniform", 128), ("hot4", 256)):
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
        verdicts.append((bias_mode, same_ids, bool(np.array_equal(got, want)), rel))
        # both forms of the exchange (a row per route / a row per destination): same bits
        from moonshine_b200.ep import ep_forward
        for form in (False, True):
            out1, ids1, _ = ep_forward(ep_layer.backend, xl, cfg, once_per_destination=form)
            torch.cuda.synchronize()
            same = bool(np.array_equal(bf16_tensor_to_bits(out1), got)) and bool(torch.equal(ids1, ids))
            verdicts.append((bias_mode + ("/row per destination" if form else "/row per route"), same, same,
                             0.0 if same else 1.0))
        # the same pass cut into two row ranges pipelined against each other: same bits
        piped = ExpertParallelLayer(cfg, seed=5, device=device, tokens=tokens, weights=weights, pieces=2)
        for _ in range(3):
            out2, ids2, _ = piped.forward(xl, want_routes=True)
        torch.cuda.synchronize()
        same = bool(np.array_equal(bf16_tensor_to_bits(out2), got)) and bool(torch.equal(ids2, ids))
        verdicts.append((bias_mode + "/pipelined", same, same, 0.0 if same else 1.0))
    ok = all(v[1] and v[3] <= 1e-3 for v in verdicts)
    sys.stderr.write(f"rank {rank}: {verdicts}\n")
    # one verdict line for the whole job (lines of several ranks could interleave)
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
