"""The per-block codec core of the CUDA library (cswap_b200/csrc/zfp_core.cuh:
byte-sliced plane transposes, table-driven group-test coding, word emitter),
compiled for the host and driven block by block, against the CPU oracle.
This checks the kernel's arithmetic without a GPU; the GPU tests check the
kernels themselves."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

import util

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def core(tmp_path_factory):
    so = str(tmp_path_factory.mktemp("core") / "libcore_host.so")
    subprocess.check_call(["g++", "-std=c++17", "-O2", "-shared", "-fPIC", "-Wno-unknown-pragmas", "-o", so,
                           os.path.join(HERE, "host_core_harness.cpp")])
    return C.CDLL(so)


def _run(core, O, a, dims, maxbits):
    nx, ny, nz = dims
    a = np.ascontiguousarray(a, dtype=np.float32)
    s = O.zfp_encode(a, nx, ny, nz, maxbits)
    nb = ((nx + 3) // 4) * max((ny + 3) // 4, 1) * max((nz + 3) // 4, 1)
    words = nb * maxbits // 32
    out = np.zeros(words + 4, dtype=np.uint32)
    core.core_encode(a.ctypes.data_as(C.c_void_p), C.c_size_t(nx), C.c_size_t(ny), C.c_size_t(nz), maxbits,
                     out.ctypes.data_as(C.c_void_p))
    sw = s.view(np.uint32)
    assert np.array_equal(out[:words], sw[:words])
    if nz:  # the slab kernel's staged encoder must produce the same words
        out2 = np.zeros(words + 4, dtype=np.uint32)
        core.core_encode_staged(a.ctypes.data_as(C.c_void_p), C.c_size_t(nx), C.c_size_t(ny), C.c_size_t(nz), maxbits,
                                out2.ctypes.data_as(C.c_void_p))
        assert np.array_equal(out2[:words], sw[:words])
    d = O.zfp_decode(s, nx, ny, nz, maxbits)
    d2 = np.zeros(a.size, dtype=np.float32)
    inw = np.zeros(words + 4, dtype=np.uint32)
    inw[:sw.size] = sw
    core.core_decode(inw.ctypes.data_as(C.c_void_p), C.c_size_t(nx), C.c_size_t(ny), C.c_size_t(nz), maxbits,
                     d2.ctypes.data_as(C.c_void_p))
    assert np.array_equal(d.view(np.uint32), d2.view(np.uint32))
    if nz:  # the slab kernel's position-based decoder
        d3 = np.zeros(a.size, dtype=np.float32)
        core.core_decode_pos(inw.ctypes.data_as(C.c_void_p), C.c_size_t(nx), C.c_size_t(ny), C.c_size_t(nz), maxbits,
                             d3.ctypes.data_as(C.c_void_p))
        assert np.array_equal(d.view(np.uint32), d3.view(np.uint32))


@pytest.mark.parametrize("dims", [(32, 32, 16), (32, 32, 7), (9, 5, 3), (4, 4, 4), (13, 0, 0), (64, 0, 0),
                                  (12, 10, 0), (32, 32, 0), (5, 5, 5)])
@pytest.mark.parametrize("maxbits", [32, 64, 96, 128, 256, 512, 1024, 2048])
def test_core_matches_oracle(core, oracle, dims, maxbits):
    nx, ny, nz = dims
    n = nx * max(ny, 1) * max(nz, 1)
    rng = np.random.default_rng(n + maxbits)
    inputs = [rng.standard_normal(n), np.tanh(rng.standard_normal(n)), np.sin(0.05 * np.arange(n)) * 3,
              rng.standard_normal(n) * (rng.random(n) < 0.1), np.full(n, 0.3),
              rng.uniform(-1, 1, n) * 10.0 ** rng.integers(-20, 20, n), np.zeros(n),
              rng.standard_normal(n) * 1e-36]
    for a in inputs:
        _run(core, oracle, a, dims, maxbits)


def test_core_on_awkward_blocks(core, oracle):
    a = util.block_zoo(32 * 32 * 12, seed=4)
    for maxbits in (64, 512, 1024):
        _run(core, oracle, a, (32, 32, 12), maxbits)


def test_stream_sizes_agree(core, oracle):
    core.core_stream_bytes.restype = C.c_size_t
    for dims in [(32, 32, 8192), (5, 5, 5), (13, 10, 0), (37, 0, 0), (1, 0, 0)]:
        for maxbits in (37, 64, 300, 512):
            got = core.core_stream_bytes(C.c_size_t(dims[0]), C.c_size_t(dims[1]), C.c_size_t(dims[2]), maxbits)
            assert got == oracle.zfp_stream_bytes(*dims, maxbits)


@pytest.mark.parametrize("maxbits", [32, 64, 128, 512, 1024])
def test_decoders_agree_on_arbitrary_streams(core, oracle, maxbits):
    """Decoding is defined for any bit string (a swapped-out tensor may come
    back from a file): both decoders of the library's core must produce what
    the oracle produces, bit for bit, also for streams no encoder wrote."""
    nx, ny, nz = 32, 32, 8
    nb = 8 * 8 * 2
    words = nb * maxbits // 32
    for sw in util.arbitrary_streams(words, maxbits):
        s64 = np.zeros((words + 1) // 2, dtype=np.uint64)
        s64.view(np.uint32)[:words] = sw
        d = oracle.zfp_decode(s64, nx, ny, nz, maxbits)
        inw = np.zeros(words + 4, dtype=np.uint32)
        inw[:words] = sw
        for fn in (core.core_decode, core.core_decode_pos):
            out = np.zeros(nx * ny * nz, dtype=np.float32)
            fn(inw.ctypes.data_as(C.c_void_p), C.c_size_t(nx), C.c_size_t(ny), C.c_size_t(nz), maxbits,
               out.ctypes.data_as(C.c_void_p))
            assert np.array_equal(d.view(np.uint32), out.view(np.uint32))
