"""The CPU oracle against what the reference's own CUDA kernels produced on a
B200 (tests/golden/ref_cuda_golden.npz, written by
tests/golden/make_ref_cuda_golden.py).  Runs without a GPU."""
import hashlib
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_ref_cuda_golden as G  # noqa: E402

PATH = os.path.join(HERE, "golden", "ref_cuda_golden.npz")
if not os.path.exists(PATH):
    pytest.skip("ref_cuda_golden.npz has not been generated", allow_module_level=True)
GOLD = np.load(PATH)


def _sha(a):
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(a).tobytes()).digest(), dtype=np.uint8)


@pytest.mark.parametrize("case", G.CASES, ids=[c[0] for c in G.CASES])
def test_zfp_small_fields(oracle, case):
    name, dims, maxbits, gen, seed = case
    nx, ny, nz = dims
    a = G.make_input(gen, nx * ny * nz, seed)
    s = oracle.zfp_encode(a, nx, ny, nz, maxbits)
    assert np.array_equal(s, GOLD[f"{name}.stream"])
    back = oracle.zfp_decode(s, nx, ny, nz, maxbits)
    assert np.array_equal(back.view(np.uint32), GOLD[f"{name}.decoded"].view(np.uint32))


@pytest.mark.parametrize("case", G.BIG, ids=[c[0] for c in G.BIG])
def test_zfp_benchmark_tensor_digest(oracle, case):
    name, dims, maxbits, gen, seed = case
    nx, ny, nz = dims
    a = G.make_input(gen, nx * ny * nz, seed)
    s = oracle.zfp_encode(a, nx, ny, nz, maxbits, threads=oracle.max_threads())
    assert np.array_equal(_sha(s), GOLD[f"{name}.stream_sha256"])
    back = oracle.zfp_decode(s, nx, ny, nz, maxbits, threads=oracle.max_threads())
    assert np.array_equal(_sha(back), GOLD[f"{name}.decoded_sha256"])


@pytest.mark.parametrize("case", G.SPARSE, ids=[c[0] for c in G.SPARSE])
def test_sparse_reference_layout(oracle, case):
    import util
    name, n, zf, seed = case
    a = util.relu_normal(n, zf, seed)
    P = 512 * 32
    begin, bitmap, values, nnz = oracle.legacy_sparse_compress(a, P)
    assert nnz == int(GOLD[f"{name}.nnz"][0])
    pack = begin.tobytes() + bitmap.tobytes() + values.tobytes()
    assert np.array_equal(np.frombuffer(hashlib.sha256(pack).digest(), dtype=np.uint8), GOLD[f"{name}.packed_sha256"])
    out = oracle.legacy_sparse_decompress(values, n, P, bitmap, begin, prefill=7.0)
    assert np.array_equal(_sha(out), GOLD[f"{name}.restored_sha256"])
