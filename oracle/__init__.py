"""CPU oracle for the sparse entmax decode step. TEST INFRASTRUCTURE ONLY.

This package restates, on the CPU (torch-CPU / numpy, fp32 and fp64), the
algorithm of the reference project's decode hot path:

    PagedKVCache.initialize / append      entmaxkv/kv_cache.py:40-116
    page criticality + top-k + pack       entmaxkv/kernels/page_criticality.py:24-104,
                                          entmaxkv/attention_topk.py:39-71
    Gaussian score moments                entmaxkv/kernels/gaussian_page_stats.py:8-121,
                                          entmaxkv/gaussian_utils.py:66-200
    single-Gaussian tau solver            entmaxkv/tau_solver.py:210-273,
                                          entmaxkv/kernels/tau_solver_gpu.py:79-125
    threshold select + pack, seqlens      entmaxkv/kernels/selection_pack.py:7-20,113-198
    tau clamp                             entmaxkv/kernels/tau_clamp.py:8-73
    paged exact entmax decode             entmaxkv/kernels/adadecode_paged.py:39-507,
                                          entmaxkv/kernels/adadecode.py:12-112,381-426
    paged fixed/corrected-tau decode      entmaxkv/kernels/adadecode_paged_gaussian_tau.py:12-175
    page-mixture tau solver               entmaxkv/kernels/tau_solver_page_mixture.py:67-185
    dense entmax decode (tests' oracle)   tests/benchmark_utils.py:56-83

Nothing in the product package imports it.  Only the test-suite, the smoke
check and the benchmark's CPU-baseline / reference arm execute it, and there
only as the checker or as the timed CPU baseline.

Parity pin: the parts of the reference that run without a GPU (cache
statistics, torch criticality, torch Gaussian statistics, the CPU tau
solvers, the CPU branch of the tau clamp, the page-mixture solver) were run
in a CPU container and their outputs committed under ``tests/golden/``
together with the generating script; ``tests/test_oracle_golden.py`` checks
this oracle against them.  The Triton-only parts of the reference (page
scores in the query dtype, top-k tables, threshold select/pack with token
counts, the tau clamp and the two paged decodes) were run unmodified on a
B200; their outputs are ``tests/golden/ref_triton.npz`` (generating script
beside it) and ``tests/test_oracle_triton_golden.py`` checks this oracle
against them: selections identical, fp32 cases to 1e-5, 16-bit cases to the
rounding of the reference's 16-bit dot products.
"""

from . import cache, topk, gaussian, decode, dense  # noqa: F401
