"""The C-ABI library: it loads, exports every symbol the public header declares,
and refuses to compute without a GPU (no CPU fallback)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from ornithology_b200 import _lib, build
    build.build()
    return _lib.load()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "ornith_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"\b(ornith_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_header_symbols_are_exported(lib):
    names = declared_symbols()
    assert len(names) >= 40
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared in include/ornith_cuda.h but not exported: {missing}"


def test_binding_table_matches_header(lib):
    from ornithology_b200 import _lib
    assert sorted(_lib.SYMBOLS) == declared_symbols()


def test_struct_layouts_match_the_engine(lib):
    from ornithology_b200 import _lib
    # reference: src/ornith_attn.h:57-69 -> 6 pointers + 5 ints on LP64
    assert C.sizeof(_lib.KvCache) == 6 * 8 + 5 * 4 + 4
    assert _lib.KvCache.quantized.offset == 48 and _lib.KvCache.len.offset == 56
    assert C.sizeof(_lib.DeltaState) == 16 and C.sizeof(_lib.ConvState) == 16
    assert lib.ornith_kv_bytes_per_token(2, 256, 0) == 4096
    assert lib.ornith_kv_bytes_per_token(2, 256, 1) == 1040


def test_no_cpu_fallback_without_a_gpu(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    assert lib.ornith_backend_cuda_available() == 0
    p = C.c_void_p()
    assert lib.ornith_cuda_malloc(C.byref(p), 64) == 6          # ORNITH_ERR_BACKEND
    assert b"no CPU fallback" in lib.ornith_cuda_last_error()
    from ornithology_b200 import attn
    import numpy as np
    # tier 1 keeps struct handling alive but computes nothing: outputs stay untouched
    c = attn.kv_init(4, 1, 8)
    out = np.full(8, 7.0, np.float32)
    z = np.ones(8, np.float32)
    attn.gqa_step(c, z, z, z, 1, out=out)
    assert (out == 7.0).all() and c.len == 0
    attn.kv_free(c)


def test_decode_scratch_follows_the_batch(lib):
    """Host-side sizing only (no GPU work).  The size query does not see the cache, so it covers both schedules:
    the grid of splits (finer splits, hence more partials per head, when the batch is too small to fill the GPU;
    the CUDA-core kernel's 512-token splits as a floor) and the balanced ranges of the Q8_0 raw-fragment kernel
    (one partial slot per head for each of at most 592 / head-group-columns ranges plus one per sequence)."""
    from ornithology_b200._lib import CudaFullLayer
    layer = CudaFullLayer(16, 2, 256, 64, 1, 1e-6, 0.0, None, None, None)

    def rows(n_seq, max_len):
        total = lib.ornith_cuda_full_attn_step_scratch(C.byref(layer), n_seq, max_len)
        fixed = (n_seq * 16 * 256 * 4 + 255) // 256 * 256 + (n_seq * 16 * 4 + 255) // 256 * 256
        return (total - fixed) / (16 * 258 * 4)                          # partial rows per head

    def balanced(n_seq, max_len):
        tiles = -(-max_len // 16)
        floor_w = max(16, -(-tiles // 32))
        return min(592 // 2, -(-n_seq * tiles // floor_w)) + n_seq

    # 64 sequences of up to 32k tokens: the 512-token splits of the CUDA-core path (65 per sequence) bound it
    assert abs(rows(64, 32832) - 64 * 65) < 0.1 and balanced(64, 32832) == 296 + 64
    # 4 sequences x 8k: 320-token splits -> 26 partials per (sequence, head) = 104 rows; balanced: 122 ranges + 4
    assert abs(rows(4, 8256) - max(4 * 26, balanced(4, 8256))) < 0.1 and balanced(4, 8256) == 126
    # 8 sequences x 16k: 576-token splits -> 29, below the CUDA-core path's 33 -> 264 rows; balanced: 249 + 8
    assert abs(rows(8, 16448) - max(8 * 33, balanced(8, 16448))) < 0.1
    assert lib.ornith_cuda_full_attn_step_scratch(C.byref(layer), 0, 100) == 0


def test_product_does_not_touch_the_oracle():
    """Nothing under the package or include/ may reference oracle/."""
    pkg = os.path.join(ROOT, "ornithology_b200")
    for dirpath, _, files in os.walk(pkg):
        if "build" in dirpath.split(os.sep)[-1:]:
            continue
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".c", ".h")):
                text = open(os.path.join(dirpath, f), errors="replace").read()
                assert "oracle" not in text.lower(), f"{f} mentions the oracle"


def test_projection_sizing_and_no_gpu_behaviour(lib):
    """Host-side: the scratch of the integer projections is the Q8_K image of the activations (one 2336-byte image
    per 8 tokens x 256 inputs, the same for the three weight types), nothing for a type without an integer path or
    a width that is not a multiple of 256; without a GPU the products fail with a status."""
    import torch
    from ornithology_b200 import _lib
    img = lambda T, n_in: -(-(-(-T // 8) * (n_in // 256) * 2336) // 256) * 256
    for wt in (8, 12, 14):
        assert lib.ornith_cuda_matmul_q_scratch(wt, 1, 2048) == img(1, 2048)
        assert lib.ornith_cuda_matmul_q_scratch(wt, 70, 4096) == img(70, 4096)
    assert lib.ornith_cuda_matmul_q_scratch(13, 8, 2048) == 0          # Q5_K: the engine dequantises it
    assert lib.ornith_cuda_matmul_q_scratch(8, 8, 300) == 0
    assert lib.ornith_cuda_matmul_q_scratch(8, 0, 2048) == 0
    assert C.sizeof(_lib.CudaQproj) == 32 and _lib.CudaQproj.n_out.offset == 16 and _lib.CudaQproj.y.offset == 24
    if not torch.cuda.is_available():
        p = _lib.CudaQproj(8, None, 64, None)
        assert lib.ornith_cuda_matmul_q_group(C.byref(p), 1, 2048, None, 4, 0, None) != 0
        assert lib.ornith_cuda_matmul_q(8, None, 2048, 64, None, 0, 4, None, 0, None, 0, None) != 0
