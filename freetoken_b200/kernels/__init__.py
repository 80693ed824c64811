"""Hand-written CUDA kernels for sm_100a behind a C ABI (:mod:`ops`), and their build (:mod:`library`)."""
