"""CPU-side checks of the C ABI: the shared library builds for sm_100a without a GPU, loads,
exports every function the header declares, and the ctypes binding covers them all.
No compute entry point is called here."""

import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "entmaxkv_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ekv_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib_path():
    from entmaxkv_b200.build import build_library
    return build_library()


def test_header_declares_the_expected_surface():
    names = declared_functions()
    for must in ("ekv_page_stats_init", "ekv_append", "ekv_topk_select", "ekv_gaussian_moments",
                 "ekv_gaussian_select", "ekv_decode", "ekv_decode_scores", "ekv_decode_values"):
        assert must in names


def test_library_exports_every_declared_symbol(lib_path):
    lib = ctypes.CDLL(lib_path)
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert not missing, f"declared in the header but not exported: {missing}"


def test_ctypes_binding_covers_the_header(lib_path):
    from entmaxkv_b200 import _lib
    assert sorted(_lib.SIGNATURES) == declared_functions()
    lib = _lib.load()
    assert lib.ekv_version() >= 100
    # pure host-side queries may be called without a GPU
    assert lib.ekv_work_items_per_head(4097) == 17
    assert lib.ekv_decode_workspace_bytes(1, 1, 128, 256) > 256 * 4
    assert lib.ekv_gaussian_workspace_bytes(2, 4, 1000) > 0
    assert lib.ekv_decode_workspace_bytes(0, 1, 128, 256) == 0


def test_argument_checks_answer_on_the_host_without_a_gpu():
    """Host-side refusals return EKV_ERR_ARG (-2) before anything is launched: null and misaligned buffers of the
    input staging call, a null counter, a null descriptor of the small-problem query; and the status bits are
    the header's."""
    from entmaxkv_b200 import _lib
    lib = _lib.load()
    buf = (ctypes.c_char * 256)()
    base = ctypes.addressof(buf)
    base += (-base) % 16
    assert lib.ekv_stage_inputs(None, base, 16, base, base, 16, base, base, 16, None) == -2
    assert lib.ekv_stage_inputs(base, base + 2, 16, base, base, 16, base, base, 16, None) == -2     # misaligned source
    assert lib.ekv_stage_inputs(base, base, 24, base, base, 16, base, base, 16, None) == -2         # size not a multiple of 16
    assert lib.ekv_copy_timeouts(None) == -2
    assert lib.ekv_topk_decode_fused_supported(None, 4, 64, 1024, 2) == 0
    text = open(HEADER).read()
    bits = dict(re.findall(r"(EKV_STATUS_[A-Z_]+)\s*=\s*(\d+)", text))
    assert bits == {"EKV_STATUS_PAGE_RANGE": "1", "EKV_STATUS_CAPACITY": "2", "EKV_STATUS_TOKENS": "4",
                    "EKV_STATUS_PEER_TIMEOUT": "8", "EKV_STATUS_COPY_TIMEOUT": "16"}


def test_cache_descriptor_layout_matches_the_header():
    """Field order and types of the ctypes struct follow ekv_cache_desc."""
    from entmaxkv_b200 import _lib
    text = open(HEADER).read()
    start = text.index("typedef struct ekv_cache_desc {") + len("typedef struct ekv_cache_desc {")
    body = text[start:text.index("} ekv_cache_desc;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = []
    for decl in body.split(";"):
        decl = decl.strip()
        m = re.match(r"(?:const\s+)?(void\*|int32_t\*|int64_t|int32_t)\s+(.*)", decl)
        if m:
            fields += [f.strip() for f in m.group(2).split(",")]
    assert [n for n, _ in _lib.CacheDesc._fields_] == fields
    assert ctypes.sizeof(_lib.CacheDesc) == 7 * 8 + 4 * 8 + 8 * 4 + 3 * 8 + 2 * 4


def test_product_refuses_cpu_tensors_instead_of_falling_back():
    import torch
    import entmaxkv_b200 as E
    c = E.PagedKVCache(16)
    with pytest.raises(ValueError):
        c.initialize(torch.zeros(1, 1, 16, 64), torch.zeros(1, 1, 16, 64))
    # nothing under the product package imports the oracle
    pkg = os.path.join(ROOT, "entmaxkv_b200")
    for fn in os.listdir(pkg):
        if fn.endswith(".py"):
            src = open(os.path.join(pkg, fn)).read()
            assert not re.search(r"^\s*(import|from)\s+oracle", src, flags=re.M), fn


def test_group_shared_route_is_taken_only_for_the_shapes_its_kernels_cover(monkeypatch):
    """Host logic of the Gaussian-aware wrapper: GQA groups of four, 16-bit, head_dim 128, page size
    a power of two in 4..32 and no ALiBi go through the group-shared K pass; everything else, and
    EKV_GROUPED=0, keeps one page table per query head."""
    import torch
    from entmaxkv_b200.attention_gaussian import grouped_enabled

    class FakeCache:
        def __init__(self, kv_heads, dtype=torch.bfloat16, page_size=16, page_capacity=8192, D=128):
            self._k = torch.empty(1, kv_heads, 1, D, dtype=dtype)
            self.page_size = page_size
            self.page_capacity = page_capacity

    def q(heads, D=128):
        return torch.empty(1, heads, 1, D, dtype=torch.bfloat16)

    monkeypatch.delenv("EKV_GROUPED", raising=False)
    assert grouped_enabled(q(32), FakeCache(8))
    assert grouped_enabled(q(4), FakeCache(1, dtype=torch.float16, page_size=4))
    assert not grouped_enabled(q(32), FakeCache(32))                       # MHA
    assert grouped_enabled(q(64), FakeCache(8))                            # groups of eight
    assert not grouped_enabled(q(16), FakeCache(8))                        # groups of two
    assert not grouped_enabled(q(64), FakeCache(8, page_capacity=200000))  # eight bitmaps would not fit
    assert not grouped_enabled(q(32), FakeCache(8, dtype=torch.float32))   # fp32 cache
    assert not grouped_enabled(q(32, 64), FakeCache(8, D=64))              # head_dim 64
    assert not grouped_enabled(q(32), FakeCache(8, page_size=64))
    assert not grouped_enabled(q(32), FakeCache(8, page_size=24))
    assert not grouped_enabled(q(32), FakeCache(8, page_capacity=400000))  # bitmaps would not fit shared memory
    assert not grouped_enabled(q(32), FakeCache(8), alibi=(object(), None))
    monkeypatch.setenv("EKV_GROUPED", "0")
    assert not grouped_enabled(q(32), FakeCache(8))


def test_device_alias_refuses_memory_the_device_cannot_address():
    """The host-to-host step stores its output through a device alias of a page-locked host tensor; pageable or
    strided host memory is refused on the host, before any kernel gets the pointer."""
    import torch
    from entmaxkv_b200.graph import device_alias
    with pytest.raises(ValueError):
        device_alias(torch.empty(8, 16))                      # pageable
    with pytest.raises(ValueError):
        device_alias(torch.empty(8, 16)[:, ::2])              # strided view
