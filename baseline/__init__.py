"""Unfused comparator: the same decoder in plain PyTorch (library GEMMs, SDPA attention, NCCL all-reduce).

It exists to give the custom-kernel engine a same-box, same-shape baseline: no hand-written kernel, no fusion,
no CUDA graph tricks beyond what `torch` offers out of the box.  `bench.py --impl torch` runs it.
"""
