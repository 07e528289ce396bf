"""ornithology_b200 — B200-native CUDA backend for ornithology's attention stack.

`attn`   host-side mirror of the engine's attention header (drop-in tier)
`device` device-resident layer API (what the engine's layer wiring calls)
`build`  compiles libornith_cuda.so for sm_100a

Importing the package does not load the shared library; the first call does, and
fails loudly if it is missing.
"""
__all__ = ["attn", "device", "build", "_lib"]
