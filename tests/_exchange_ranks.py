"""Child-process body of the two-rank exchange test (launched by torch.distributed.run).

Each rank holds one contiguous range of pages of the same seeded request and runs the
Gaussian step three ways: sequence-sharded with the reductions fused over peer memory,
sequence-sharded with NCCL all-reduces, and (rank 0) unsharded on one GPU.  A rank leaves
only between steps, after a barrier; NVLS is off in the environment of the launcher.
"""

import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    import entmaxkv_b200 as E
    from entmaxkv_b200 import sharded
    from entmaxkv_b200.exchange import PeerExchange
    from tests import _harness as H

    rank, local, world = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    B, Hq, Hkv, D, S, P = 1, 16, 2, 128, 512 * 16 + 5, 16
    inp = H.to_cuda(H.cpu_inputs(B, Hq, Hkv, D, S, torch.bfloat16, seed=97, needle_pages=(5, 300)))
    lo, hi = sharded.split_pages(S, P, world)[rank]

    def fresh_shard():
        sh = sharded.GpuSequenceShard(P, rank, world)
        sh.initialize(inp["k"][:, :, lo:hi].contiguous(), inp["v"][:, :, lo:hi].contiguous(), capacity=hi - lo + 64)
        sh.set_global_lengths([S] * B)
        return sh

    x = PeerExchange(rank, world, max_floats=1 << 14)
    a, b = fresh_shard(), fresh_shard()
    args = ([inp["q"]], [inp["k_new"]], [inp["v_new"]])
    outs_x, outs_n = [], []
    for step in range(3):                       # three steps: both parities of every slot, growing cache
        outs_x.append(sharded.sharded_gaussian_decode_step([a], None, *args, alpha=1.5, exchange=x)[0].clone())
        outs_n.append(sharded.sharded_gaussian_decode_step([b], sharded.dist_reduce(), *args, alpha=1.5)[0].clone())
    torch.cuda.synchronize()
    x.check()
    for ox, on in zip(outs_x, outs_n):
        # both reduce fp32 partials; the fused step scores the rows of a GQA group once with tensor-core tiles
        # (fp32 accumulation of the same exact products in another order), the NCCL formulation per head
        scale = max(1.0, float(on.abs().max()))
        np.testing.assert_allclose(ox.cpu().numpy(), on.cpu().numpy(), rtol=0, atol=1e-4 * scale)
    np.testing.assert_allclose(a.tau.cpu().numpy(), b.tau.cpu().numpy(), rtol=2e-5, atol=1e-6)
    assert torch.equal(a.counts, b.counts) and torch.equal(a.tokens, b.tokens)
    # every rank holds bit-identical results of the fused exchange
    mine = outs_x[-1].contiguous()
    everyone = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(everyone, mine)
    assert all(torch.equal(everyone[0], t) for t in everyone)
    # bf16 output written by the exchange kernel itself
    c = fresh_shard()
    out16 = torch.zeros(B, Hq, 1, D, dtype=torch.bfloat16, device="cuda")
    sharded.sharded_gaussian_decode_step([c], None, *args, alpha=1.5, exchange=x, out=out16)
    assert torch.equal(out16, outs_x[0].to(torch.bfloat16))      # executions are bit-reproducible
    # graph replay of the fused step
    d = fresh_shard()
    g = sharded.ShardedStepGraph(d, None, Hq, alpha=1.5, exchange=x)
    for step in range(3):
        og = g.step(inp["q"], inp["k_new"], inp["v_new"])
        torch.cuda.synchronize()
        assert torch.equal(og, outs_x[step]), step
    g.release()
    # the same with the inputs in page-locked host buffers and the copies in and out as nodes of the graph
    e = fresh_shard()
    g2 = sharded.ShardedStepGraph(e, None, Hq, alpha=1.5, exchange=x)
    io = g2.pinned_io()
    for name in ("q", "k_new", "v_new"):
        io[name].copy_(inp[name])
    for step in range(3):
        og = g2.step_pinned()
        torch.cuda.synchronize()
        assert torch.equal(og, outs_x[step].cpu()), step
    g2.release()
    x.check()
    if rank == 0:
        cache = E.PagedKVCache(P)
        cache.initialize(inp["k"], inp["v"])
        out = torch.zeros_like(inp["q"])
        E.sparse_attention_decode_gaussian_aware_entmax(inp["q"], cache, inp["k_new"], inp["v_new"], out,
                                                        append_cache=True)
        ref = out[:, :, 0].float().cpu().numpy()
        got = outs_x[0][:, :, 0].cpu().numpy()
        scale = max(1.0, float(np.abs(ref).max()))
        assert np.abs(ref - got).max() <= 2e-3 * scale + 0.5 * 2 ** -8 * np.abs(got).max()
    torch.cuda.synchronize()
    dist.barrier()
    x.close()
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print("EXCHANGE-RANKS-OK")


if __name__ == "__main__":
    main()
