"""CPU oracle for the subgame-solving hot path.

TEST INFRASTRUCTURE ONLY.  These modules restate, on the CPU, the algorithms of the
upstream P2 implementation so that the CUDA kernels can be checked against them and so
that a CPU baseline can be timed beside the GPU numbers.  Only the test-suite, the smoke
check and the CPU-baseline leg of the benchmark may import this package; the product
package never does and has no CPU fallback.

Parity is pinned: every module here is checked against golden vectors produced by running
the upstream code itself (see tests/golden/make_golden.py and tests/test_oracle_*.py).
"""
