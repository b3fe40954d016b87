"""CPU oracle for the KV-cache hot path.  TEST INFRASTRUCTURE ONLY.

Everything in this package is a CPU restatement of the reference
(MorphServe / SwiftLLM worker) algorithm for one path: paged-attention decode,
KV append (store_kvcache), block-table maintenance, elastic pool resize and
block swap.  It exists so the CUDA path can be checked against it.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark
may import it.  The product package never does: it fails loudly when its CUDA
library is missing instead of falling back to anything here.

Parity pinning: the reference ships no golden vectors or tests.  The oracle is
pinned against outputs of the reference's own kernels executed in the Triton
interpreter on CPU; the fixtures and the script that made them live in
``tests/golden/``.
"""
