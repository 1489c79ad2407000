"""Launched by tests/test_cuda_ep.py under torchrun with 2 or more ranks (one GPU each): the expert-parallel
layer on a sharded token set must equal the single-GPU layer on the same tokens.  Prints "EP_OK" per rank."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

import __graft_entry__ as entry  # noqa: E402
from oracle import quant  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pkg = entry.load_package()
    dims = dict(H=1280, E=64, K=6, F=896, S=1792)
    rng = np.random.default_rng(4)
    bias = quant.zipf_logit_bias(rng, 64)
    L = quant.synth_layer(rng, expert_qtype=quant.QTYPE_Q4_0, logit_bias=bias, **dims)
    n_total = 96 * world + 8                                   # ragged: the last rank gets 8 more tokens
    hidden_all = quant.synth_activations(rng, n_total, dims["H"])
    resid_all = quant.synth_activations(rng, n_total, dims["H"])
    lo = 96 * rank
    hi = n_total if rank == world - 1 else 96 * (rank + 1)
    with pkg.Context() as ctx:
        ctx.map_layer(L)
        ctx.allocate_runtime_arenas(n_total)                   # a rank may receive every pair
        ctx.set_stream(torch.cuda.current_stream().cuda_stream)
        d_all = torch.from_numpy(hidden_all).cuda().view(torch.float16)
        r_all = torch.from_numpy(resid_all).cuda().view(torch.float16)
        want = torch.zeros_like(d_all)
        ctx.layer_forward(0, d_all, n_total, want, residual=r_all)          # single-GPU answer for all tokens
        ctx.synchronize()
        layer = pkg.ep.ExpertParallelLayer(ctx, 0, dims["E"], dims["K"], dims["H"], rank=rank, world=world, dist_module=dist)
        mine = d_all[lo:hi].contiguous()
        out = torch.zeros_like(mine)
        plan = layer.forward(mine, out, residual=r_all[lo:hi].contiguous())
        ctx.synchronize()
        torch.cuda.synchronize()
        same = torch.equal(out, want[lo:hi])
        diff = float((out.float() - want[lo:hi].float()).abs().max())
        # the same layer with the exchange over peer memory (CUDA IPC mappings of the other ranks' buffers)
        peer = pkg.ep.PeerExpertParallelLayer(ctx, 0, dims["E"], dims["K"], dims["H"], row_capacity=n_total * dims["K"],
                                              rank=rank, world=world, dist_module=dist)
        for call in (peer.forward, peer.forward_collectives, peer.forward_host_counts, peer.forward):   # ranks synchronised on the device / by collectives / offsets on the host
            out2 = torch.zeros_like(mine)
            call(mine, out2, residual=r_all[lo:hi].contiguous())
            ctx.synchronize()
            torch.cuda.synchronize()
            same = same and torch.equal(out2, want[lo:hi]) and peer.last_plan.rows_received == plan.rows_received
        dist.barrier()
        peer.close()
        print(f"rank {rank}: rows received {plan.rows_received}, max diff {diff:.3e}, {'EP_OK' if same else 'EP_MISMATCH'}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if same else 1)


if __name__ == "__main__":
    main()
