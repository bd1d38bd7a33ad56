"""svod_b200 — a B200 (sm_100a) implementation of svod's `tk` encoder hot path.

`svod_b200.ops` mirrors `svod_tk::ops`; `svod_b200.encoders` holds the three
encoder stacks that call it; the CUDA kernels and the C ABI live in `csrc/` and
are built into `lib/libsvodb.so` by `python -m svod_b200.build`.
"""
__version__ = "0.1.0"
