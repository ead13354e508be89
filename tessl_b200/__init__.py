"""tessl_b200: the MLX affine-quantized matmul path of bharathvbcr/tessl on NVIDIA B200.

`tessl_b200.nn` mirrors the reference's operator API over the C ABI of
`libtessl_b200.so` (hand-written sm_100a kernels, built in-tree by
`python -m tessl_b200.build`); `tessl_b200.synth` draws the seeded synthetic
tensors benchmarks and tests use; `tessl_b200.sharded` column-shards a bank
across GPUs. There is no CPU or PyTorch fallback: the first operator call
raises if the library is missing.
"""
__all__ = ["capi", "nn", "synth"]
