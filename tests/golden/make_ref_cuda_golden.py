"""Generates tests/golden/ref_cuda_golden.npz from the REFERENCE'S OWN CUDA
KERNELS run on a GPU (oracle/_ref/libcswap_ref_cuda.so, built by
oracle/build_ref_cuda.sh where the reference tree is mounted).

    python tests/golden/make_ref_cuda_golden.py [output.npz]

Needs a CUDA device.  Inputs are regenerated from seeds by the tests; only what
the reference's kernels produced is stored: whole streams and decoded arrays
for small fields, SHA-256 digests for the 32 MiB benchmark tensor.  These pin
the CPU oracle to the reference's GPU path, including blocks whose planes are
written as full 64-bit words (the case a host build of the reference's bit
writer cannot reproduce).
"""
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(HERE))

SLACK = 4096

# name, (nx, ny, nz), maxbits, generator in tests/util.py, seed
CASES = [
    ("tanh_rate8", (32, 32, 16), 512, "tanh_normal", 301),
    ("normal_rate4", (32, 32, 8), 256, "normal", 302),
    ("normal_rate16", (32, 32, 8), 1024, "normal", 303),
    ("uniform_rate8", (32, 32, 8), 512, "uniform", 304),
    ("zoo_64bits", (32, 32, 8), 64, "block_zoo", 305),
    ("zoo_rate8", (32, 32, 8), 512, "block_zoo", 306),
    ("zoo_rate16", (32, 32, 8), 1024, "block_zoo", 307),
    ("zoo_rate32", (32, 32, 8), 2048, "block_zoo", 308),
    ("partial_30x17x9", (30, 17, 9), 512, "normal", 309),
    ("partial_z_32x32x6", (32, 32, 6), 512, "tanh_normal", 310),
]
# digests only
BIG = [("config1_tanh_rate8", (32, 32, 8192), 512, "tanh_normal", 1)]
SPARSE = [("sparse_c2_75", 128 * 128 * 16 * 16, 0.75, 3), ("sparse_ragged", 70001, 0.5, 4)]


def make_input(gen, n, seed):
    import util
    return getattr(util, gen)(n, seed)


def stream_bytes(dims, maxbits):
    nx, ny, nz = dims
    blocks = ((nx + 3) // 4) * ((max(ny, 1) + 3) // 4) * ((max(nz, 1) + 3) // 4)
    return (blocks * maxbits + 63) // 64 * 8


def main(out_path):
    import torch
    from oracle import oracle as O
    R = O.ref_cuda()
    out = {}

    def run(dims, maxbits, a):
        nx, ny, nz = dims
        nbytes = stream_bytes(dims, maxbits)
        t = torch.from_numpy(a).cuda()
        buf = torch.zeros(nbytes + SLACK, dtype=torch.uint8, device="cuda")
        torch.cuda.synchronize()
        R.refcuda_zfp_compress(t.data_ptr(), nx, ny, nz, maxbits, buf.data_ptr(), buf.numel())
        back = torch.zeros(a.size, dtype=torch.float32, device="cuda")
        R.refcuda_zfp_decompress(buf.data_ptr(), buf.numel(), nx, ny, nz, maxbits, back.data_ptr())
        torch.cuda.synchronize()
        return buf[:nbytes].cpu().numpy().view(np.uint64), back.cpu().numpy()

    for name, dims, maxbits, gen, seed in CASES:
        nx, ny, nz = dims
        a = make_input(gen, nx * ny * nz, seed)
        s, b = run(dims, maxbits, a)
        out[f"{name}.stream"] = s
        out[f"{name}.decoded"] = b
    for name, dims, maxbits, gen, seed in BIG:
        nx, ny, nz = dims
        a = make_input(gen, nx * ny * nz, seed)
        s, b = run(dims, maxbits, a)
        out[f"{name}.stream_sha256"] = np.frombuffer(hashlib.sha256(s.tobytes()).digest(), dtype=np.uint8)
        out[f"{name}.decoded_sha256"] = np.frombuffer(hashlib.sha256(b.tobytes()).digest(), dtype=np.uint8)
    for name, n, zf, seed in SPARSE:
        import util
        a = util.relu_normal(n, zf, seed)
        dimsize, blocksize = 512, 32
        P = dimsize * blocksize
        chunk = -(-n // P)
        t = torch.from_numpy(a).cuda()
        begin = torch.zeros(P, dtype=torch.int32, device="cuda")
        num = torch.zeros(1, dtype=torch.int32, device="cuda")
        bitmap = torch.zeros(P * (-(-chunk // 32)), dtype=torch.int32, device="cuda")
        values = torch.zeros(n, dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        nnz = R.refcuda_sparse_compress(t.data_ptr(), n, dimsize, blocksize, begin.data_ptr(), num.data_ptr(),
                                        bitmap.data_ptr(), values.data_ptr())
        restored = torch.full((n,), 7.0, dtype=torch.float32, device="cuda")
        R.refcuda_sparse_decompress(values.data_ptr(), restored.data_ptr(), n, dimsize, blocksize,
                                    bitmap.data_ptr(), begin.data_ptr())
        torch.cuda.synchronize()
        pack = begin.cpu().numpy().tobytes() + bitmap.cpu().numpy().tobytes() + values[:nnz].cpu().numpy().tobytes()
        out[f"{name}.nnz"] = np.array([nnz], dtype=np.int64)
        out[f"{name}.packed_sha256"] = np.frombuffer(hashlib.sha256(pack).digest(), dtype=np.uint8)
        out[f"{name}.restored_sha256"] = np.frombuffer(
            hashlib.sha256(restored.cpu().numpy().tobytes()).digest(), dtype=np.uint8)
    np.savez_compressed(out_path, **out)
    print(f"wrote {out_path}: {len(out)} arrays")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "ref_cuda_golden.npz"))
