"""The allocation-free append entry point against the regular one (run on a B200: ``-m gpu``).

``ekv_append_static`` is for hosts that cannot give the library scratch memory - their
device memory was carved up at start-up, or the step runs where cudaMalloc is not allowed.
It must leave the cache exactly as ``ekv_append`` does.  This file sorts last on purpose,
so a run that stops at the first failure has already been through every other test; it
also passes when run on its own in a fresh process.
"""

import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _cache_pair(B, Hkv, D, S, dtype, seed):
    import entmaxkv_b200 as E
    g = torch.Generator().manual_seed(seed)
    k = torch.randn(B, Hkv, S, D, generator=g).to(dtype).cuda()
    v = torch.randn(B, Hkv, S, D, generator=g).to(dtype).cuda()
    a, b = E.PagedKVCache(16), E.PagedKVCache(16)
    a.initialize(k, v)
    b.initialize(k, v)
    return a, b, g


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_static_append_matches_regular_append_on_consecutive_calls(dtype):
    from entmaxkv_b200 import _lib
    lib = _lib.load()
    B, Hkv, D, S = 3, 4, 128, 45
    ref, dut, g = _cache_pair(B, Hkv, D, S, dtype, seed=91)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for step in range(5):               # 45 -> 50: fills a page and starts the next one
        kn = torch.randn(B, Hkv, 1, D, generator=g).to(dtype).cuda()
        vn = torch.randn(B, Hkv, 1, D, generator=g).to(dtype).cuda()
        ref.append(kn, vn)              # regular entry point (scratch owned by the cache object)
        rc = lib.ekv_append_static(C.byref(dut.desc()), kn.data_ptr(), vn.data_ptr(), kn.stride(0),
                                   kn.stride(1), status.data_ptr(), _lib.stream_ptr())
        assert rc == 0, f"ekv_append_static returned {rc} at step {step}"
        dut._host_lens = [n + 1 for n in dut._host_lens]
        torch.cuda.synchronize()
        assert torch.equal(dut.seq_lens, ref.seq_lens)
        assert torch.equal(dut.k_cache, ref.k_cache) and torch.equal(dut.v_cache, ref.v_cache)
        for name in ("k_min", "k_max", "k_mean", "k_std"):
            assert torch.equal(getattr(dut, name), getattr(ref, name)), (step, name)
    assert int(status.item()) == 0


def test_static_append_refuses_batches_beyond_its_built_in_scratch():
    from entmaxkv_b200 import _lib
    lib = _lib.load()
    ref, dut, g = _cache_pair(1, 2, 64, 20, torch.float16, seed=92)
    kn = torch.randn(1, 2, 1, 64, generator=g).half().cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    desc = _lib.CacheDesc.from_buffer_copy(dut.desc())
    desc.batch = 4097                   # one more than EKV_APPEND_STATIC_MAX_BATCH; refused on the host
    rc = lib.ekv_append_static(C.byref(desc), kn.data_ptr(), kn.data_ptr(), kn.stride(0), kn.stride(1),
                               status.data_ptr(), _lib.stream_ptr())
    assert rc == -5
    torch.cuda.synchronize()
    assert dut.seq_lens.tolist() == [20]
