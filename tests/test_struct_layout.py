"""The zfp object mirrors of include/cswap_compat.h against the reference's own
headers, and the reference's call sequence linked against the product library.
Needs the reference checkout (CSWAP_REFERENCE or a `reference` directory next
to the repository); skipped elsewhere.  No GPU needed: nothing is executed on
a device."""
import os
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


@pytest.fixture(scope="module")
def refdir():
    from oracle import oracle as O
    r = O.reference_root()
    if r is None:
        pytest.skip("reference checkout not present")
    return os.path.join(r, "CSWAP+")


def test_struct_sizes_and_offsets_equal_the_references(refdir, tmp_path):
    cmd = ["gcc", "-std=c11", "-w", "-c", "-I", os.path.join(refdir, "zfp"), "-I", os.path.join(ROOT, "include"),
           os.path.join(HERE, "layout_check.c"), "-o", str(tmp_path / "layout_check.o")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]


def test_reference_call_sequence_links_against_the_library(refdir, tmp_path):
    """The sequence of simple.c:40-74 (zfp_stream_open, zfp_field_3d,
    zfp_stream_maximum_size, stream_open, zfp_stream_set_bit_stream,
    zfp_stream_rewind, cuda_compress, cuda_decompress) compiled against the
    reference's zfp.h, with the reference's zfp.c and bitstream.c as the host
    helpers and libcswap_b200.so providing cuda_compress / cuda_decompress."""
    import cswap_b200
    lib = cswap_b200._lib.LIB_PATH
    if not os.path.exists(lib):
        pytest.skip("library not built")
    src = tmp_path / "calls.c"
    src.write_text('''
#include <stdlib.h>
#include "zfp.h"
size_t cuda_compress(zfp_stream*, const zfp_field*);
void cuda_decompress(zfp_stream*, zfp_field*);
int main(int argc, char** argv) {
  if (argc < 2) return 0;               /* link check only: never called without a GPU */
  float* a = malloc(32 * 32 * 8 * sizeof(float));
  zfp_field* field = zfp_field_3d(a, zfp_type_float, 32, 32, 8);
  zfp_stream* zfp = zfp_stream_open(NULL);
  zfp->minbits = zfp->maxbits = 512;
  size_t bufsize = zfp_stream_maximum_size(zfp, field);
  void* buffer = malloc(bufsize);
  bitstream* stream = stream_open(buffer, bufsize);
  zfp_stream_set_bit_stream(zfp, stream);
  zfp_stream_rewind(zfp);
  size_t n = cuda_compress(zfp, field);
  zfp_stream_rewind(zfp);
  cuda_decompress(zfp, field);
  return n == 0;
}
''')
    z = os.path.join(refdir, "zfp")
    exe = tmp_path / "calls"
    cmd = ["gcc", "-std=c99", "-w", "-I", z, str(src), os.path.join(z, "zfp.c"), os.path.join(z, "bitstream.c"),
           "-o", str(exe), "-L", os.path.dirname(lib), "-lcswap_b200", "-Wl,-rpath," + os.path.dirname(lib), "-lm"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    r = subprocess.run([str(exe)], capture_output=True, text=True)   # no argument: returns before any call
    assert r.returncode == 0, r.stderr[-1000:]
