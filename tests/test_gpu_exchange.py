"""Peer exchange of the sequence-sharded step (``ekv_exchange_*``), through the C ABI.

On one device: the single-rank degenerate case against the unfused stage calls; the data
path between two exchange objects (rank 0 runs first against a peer that has not sent yet, so
its bounded wait runs out and reports it - nothing hangs - and rank 1, run afterwards, finds
rank 0's contribution and reduces both); and with two or more GPUs, two real ranks as child
processes comparing the fused-exchange step with the NCCL step and the unsharded step.
No test here waits on a kernel that could run concurrently on the same GPU.
"""

import os
import subprocess
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_single_rank_exchange_is_identity_and_matches_unfused_stages():
    from entmaxkv_b200 import _lib
    from entmaxkv_b200.exchange import PeerExchange
    lib = _lib.load()
    x = PeerExchange(0, 1, max_floats=4096)
    g = torch.Generator(device="cuda").manual_seed(5)
    src = torch.randn(1000, generator=g, device="cuda")
    for _ in range(3):                               # both parities of the slot
        assert torch.equal(x.all_reduce(src, "sum"), src)
        assert torch.equal(x.all_reduce(src, "max", slot=1), src)
    st = _lib.stream_ptr()
    # finalize: same arithmetic as the plain stage call
    B, Hq, P = 2, 8, 16
    sums = torch.rand(B, Hq, 4, generator=g, device="cuda") * 50
    sums[..., 1] += sums[..., 0] ** 2 / 40
    lens = torch.tensor([1000, 777], dtype=torch.int32, device="cuda")
    want = torch.zeros(B, Hq, 4, device="cuda")
    got = torch.zeros_like(want)
    _lib.check(lib.ekv_gaussian_finalize_from_lengths(sums.data_ptr(), lens.data_ptr(), P, B, Hq, 1.5,
                                                      want.data_ptr(), st), "finalize")
    _lib.check(lib.ekv_exchange_gaussian_finalize(x.handle, sums.data_ptr(), lens.data_ptr(), P, B, Hq, 1.5,
                                                  got.data_ptr(), x.status.data_ptr(), st), "finalize_x")
    assert torch.equal(want, got), (want - got).abs().amax(dim=(0, 1))
    # clamp
    n = B * Hq
    tau0 = torch.rand(n, generator=g, device="cuda")
    cap = torch.rand(n, generator=g, device="cuda")
    cap[3] = -3.4e38
    floor = torch.rand(n, generator=g, device="cuda") * 0.1
    want = torch.zeros(n, device="cuda")
    _lib.check(lib.ekv_tau_clamp(tau0.data_ptr(), 1, cap.data_ptr(), floor.data_ptr(), n, 1.5, 1e-4,
                                 want.data_ptr(), st), "clamp")
    got = tau0.clone()
    _lib.check(lib.ekv_exchange_tau_clamp(x.handle, got.data_ptr(), cap.data_ptr(), floor.data_ptr(), n, 1.5, 1e-4,
                                          x.status.data_ptr(), st), "clamp_x")
    assert torch.equal(want, got)
    # Halley update
    hs = torch.rand(n, 3, generator=g, device="cuda") + 0.5
    want = tau0.clone()
    _lib.check(lib.ekv_halley_update(want.data_ptr(), hs.data_ptr(), n, 1.5, st), "halley")
    got = tau0.clone()
    _lib.check(lib.ekv_exchange_halley_update(x.handle, got.data_ptr(), hs.data_ptr(), n, 1.5,
                                              x.status.data_ptr(), st), "halley_x")
    assert torch.equal(want, got)
    # output: one rounding to the output dtype
    part = torch.randn(n, 128, generator=g, device="cuda")
    for dt in (torch.float32, torch.float16, torch.bfloat16):
        out = torch.zeros(n, 128, dtype=dt, device="cuda")
        _lib.check(lib.ekv_exchange_output(x.handle, part.data_ptr(), n, 128, out.data_ptr(), 128,
                                           _lib.dtype_code(dt), x.status.data_ptr(), st), "output_x")
        assert torch.equal(out, part.to(dt))
    x.check()
    # limits are refused on the host
    with pytest.raises(ValueError):
        x.all_reduce(torch.zeros(8192, device="cuda"))
    x.close()


def test_wait_runs_out_without_hanging_and_late_rank_sees_the_data():
    from entmaxkv_b200.exchange import PeerExchange, PeerTimeout
    r0 = PeerExchange(0, 2, max_floats=1024, connect=False)
    r1 = PeerExchange(1, 2, max_floats=1024, connect=False)
    bases = [r0.base_pointer(), r1.base_pointer()]
    r0.connect_pointers(bases)
    r1.connect_pointers(bases)
    r0.set_spin_limit(2000)                    # about a millisecond
    a = torch.arange(100, dtype=torch.float32, device="cuda")
    b = torch.full((100,), 0.5, device="cuda")
    r0.all_reduce(a, "sum")                    # peer has not sent: the wait gives up and says so
    with pytest.raises(PeerTimeout):
        r0.check()
    got = r1.all_reduce(b, "sum")              # rank 0's partial and flag are already in rank 1's inbox
    r1.check()
    assert torch.equal(got, a + b)
    r1.set_spin_limit(2000)
    r1.all_reduce(b, "max", slot=1)            # rank 0 never runs slot 1
    with pytest.raises(PeerTimeout):
        r1.check()
    # the context is intact
    assert float((a * 2).sum().item()) == float(a.sum().item()) * 2
    r0.close()
    r1.close()


def test_exchanges_with_different_grids_on_one_slot_never_take_stale_words():
    """A one-block exchange (``ekv_exchange_halley_update``) followed by the sharded decode, whose tau
    kernel trades its sums on the same slot with one block per head: the second exchange must wait for
    words of ITS number, not accept the words the first one left behind.  Two exchange objects on one
    device, rank 0 run to completion before rank 1 (rank 0's waits run out, which is reported; rank 1
    then finds all of rank 0's words and must reduce exactly them)."""
    import ctypes as C
    from entmaxkv_b200 import _lib, sharded
    from entmaxkv_b200.exchange import PeerExchange, PeerTimeout
    from tests import _harness as H
    lib = _lib.load()
    B, Hq, Hkv, D, S, P, world = 1, 8, 2, 128, 64 * 16 + 7, 16, 2
    inp = H.to_cuda(H.cpu_inputs(B, Hq, Hkv, D, S, torch.bfloat16, seed=123, needle_pages=(5, 40)))
    parts = sharded.split_pages(S, P, world)

    def make_shards():
        out = []
        for r, (lo, hi) in enumerate(parts):
            sh = sharded.GpuSequenceShard(P, r, world)
            sh.initialize(inp["k"][:, :, lo:hi].contiguous(), inp["v"][:, :, lo:hi].contiguous())
            sh.set_global_lengths([S] * B)
            out.append(sh)
        return out

    # reference: the same step with the reductions done on the host side of this process
    ref_shards = make_shards()
    sharded.sharded_gaussian_decode_step(ref_shards, sharded.local_reduce, [inp["q"]] * world,
                                         [inp["k_new"]] * world, [inp["v_new"]] * world, alpha=1.5)
    want_tau = ref_shards[0].tau.clone()

    shards = make_shards()
    for sh in shards:
        sh.append(inp["k_new"], inp["v_new"])
    sums = sharded.local_reduce([sh.moments(inp["q"], 1.5) for sh in shards], "sum")
    for sh, t in zip(shards, sums):
        sh.finalize(t)
    caps = sharded.local_reduce([sh.select() for sh in shards], "max")
    for sh, cap in zip(shards, caps):
        sh.clamp(cap)
    tau_c = shards[0].tau.clone()
    xs = [PeerExchange(r, world, max_floats=4096, connect=False) for r in range(world)]
    bases = [x.base_pointer() for x in xs]
    for x in xs:
        x.connect_pointers(bases)
    xs[0].set_spin_limit(2000)
    n = B * Hq
    g = torch.Generator(device="cuda").manual_seed(7)
    junk = [torch.rand(n, 3, generator=g, device="cuda") + 0.5 for _ in range(world)]
    side_tau0 = torch.rand(n, generator=g, device="cuda")
    side_tau = [side_tau0.clone() for _ in range(world)]
    st = _lib.stream_ptr()
    for r in range(world):
        # exchange 1 on the slot: one block, unrelated numbers
        _lib.check(lib.ekv_exchange_halley_update(xs[r].handle, side_tau[r].data_ptr(), junk[r].data_ptr(), n, 1.5,
                                                  xs[r].status.data_ptr(), st), "halley_x")
        # exchange 2 on the slot: the decode's tau kernel, one block per head
        shards[r].tau.copy_(tau_c)
        shards[r].decode_x(xs[r], 1)
        torch.cuda.synchronize()
    with pytest.raises(PeerTimeout):
        xs[0].check()                         # rank 0 ran alone: reported, nothing hung
    xs[1].check()                             # rank 1 found every word it needed
    want_side = side_tau0.clone()
    both = (junk[0] + junk[1]).contiguous()
    _lib.check(lib.ekv_halley_update(want_side.data_ptr(), both.data_ptr(), n, 1.5, st), "halley")
    assert torch.equal(side_tau[1], want_side)
    np.testing.assert_allclose(shards[1].tau.cpu().numpy(), want_tau.cpu().numpy(), rtol=1e-6, atol=1e-7)
    for x in xs:
        x.close()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("world", [2])
def test_two_ranks_fused_exchange_equals_nccl_and_unsharded(world):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29613",
           os.path.join(ROOT, "tests", "_exchange_ranks.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "EXCHANGE-RANKS-OK" in res.stdout
