"""CPU oracle for the GEMM hot path — TEST INFRASTRUCTURE, not product code.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference arm may import
this package. The product (wmma_ops_b200) never does and has no CPU path.

Parity pins
  gemm.py        restates the reference's own oracle (torch fp32 matmul on the host,
                 test_fragment_loading.py:93, benchmark_optimizations.py:112) and is pinned by
                 the reference's closed-form known-answer case (test_fragment_loading.py:225-274)
                 and by its seeded procedure (torch.manual_seed(42), :67-90).
  tile_plan.py   restates select_optimal_tile (wmma_tile_selection.hpp:30-66), pinned against
                 the reference header itself compiled with g++ (oracle/Makefile -> oracle/_ref),
                 and split_k::compute_config (wmma_xor_swizzle.hpp:293-332), which cannot be
                 compiled here (HIP header) and is pinned only by reading.
  int4.py        PARITY UNPINNED: the reference tree has no INT4 code; the format is this
                 repository's own specification.
  attention.py   PARITY UNPINNED: the reference tree documents only the signature
                 (README.md:221-251); the arithmetic is fp32 softmax(scale*Q.K^T)V.
"""
