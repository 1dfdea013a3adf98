// Host build of the per-block codec core (cswap_b200/csrc/zfp_core.cuh), used
// by the CPU test-suite to check the register-level algorithm (byte-sliced
// plane transposes, table-driven group-test coding) bit for bit against the
// oracle without a GPU.  Test scaffolding: the shipped library never runs
// the codec on the host.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <algorithm>
#include <vector>

#include "../cswap_b200/csrc/zfp_field.cuh"

namespace {
struct VecSink {
  uint32_t* w;
  void put(int i, uint32_t v) { w[i] = v; }
};
struct VecSource {
  const uint32_t* w;
  int n;
  uint32_t get(int i) const { return i < n ? w[i] : 0u; }
};
std::vector<uint32_t> enc_lut() {
  std::vector<uint32_t> t(csw::ENC_LUT_SIZE);
  for (int i = 0; i < csw::ENC_LUT_SIZE; i++) t[i] = csw::enc_lut_entry(i);
  return t;
}
std::vector<uint32_t> dec_lut() {
  std::vector<uint32_t> t(csw::DEC_LUT_SIZE);
  for (int i = 0; i < csw::DEC_LUT_SIZE; i++) t[i] = csw::dec_lut_entry(i);
  return t;
}

template <int DIMS>
void encode_field(const csw::FieldGeom& g, const float* in, int maxbits, uint32_t* out) {
  auto lut = enc_lut();
  const int nw = maxbits / 32;
  size_t nb = csw::geom_blocks(g);
  for (size_t b = 0; b < nb; b++) {
    float q[1 << (2 * DIMS)];
    csw::gather_block<DIMS>(g, in, b, q);
    VecSink s{out + b * nw};
    csw::encode_block<DIMS>(q, maxbits, s, lut.data());
  }
}
template <int DIMS>
void decode_field(const csw::FieldGeom& g, const uint32_t* in, int maxbits, float* out) {
  auto lut = dec_lut();
  const int nw = maxbits / 32;
  size_t nb = csw::geom_blocks(g);
  for (size_t b = 0; b < nb; b++) {
    float q[1 << (2 * DIMS)];
    VecSource s{in + b * nw, nw};
    csw::decode_block<DIMS>(s, maxbits, q, lut.data());
    csw::scatter_block<DIMS>(g, out, b, q);
  }
}
}  // namespace

struct HostStage {
  uint32_t* w;
  uint32_t q[csw::QUEUE_SLOTS][csw::QUEUE_FIELDS];
  void or_word(int i, uint32_t v) { w[i] |= v; }
  void q_put(int s, int f, uint32_t v) { q[s][f] = v; }
  uint32_t q_get(int s, int f) const { return q[s][f]; }
};

extern "C" {
// the staged 3-D encoder of the slab kernel (nx, ny, nz arbitrary here; whole words per block)
void core_encode_staged(const float* in, size_t nx, size_t ny, size_t nz, int maxbits, uint32_t* out) {
  csw::FieldGeom g = csw::make_geom(nx, ny, nz, 0, 0, 0);
  auto lut = enc_lut();
  const csw::PipeConsts kc = csw::pipe_consts();
  const int nw = maxbits / 32;
  std::vector<uint32_t> rows(nw + csw::STAGE_SPARE_ROWS);
  size_t nb = csw::geom_blocks(g);
  for (size_t b = 0; b < nb; b++) {
    float q[64];
    csw::gather_block<3>(g, in, b, q);
    std::fill(rows.begin(), rows.end(), 0u);
    HostStage st{rows.data(), {}};
    csw::encode_block3_staged(q, maxbits, st, lut.data(), kc);
    for (int i = 0; i < nw; i++) out[b * nw + i] = rows[i];
  }
}
// the slab kernel's position-based decoder
struct PadSource {
  const uint32_t* w;
  int n;
  uint32_t word(int i) const { return i < n ? w[i] : 0u; }
};
void core_decode_pos(const uint32_t* in, size_t nx, size_t ny, size_t nz, int maxbits, float* out) {
  csw::FieldGeom g = csw::make_geom(nx, ny, nz, 0, 0, 0);
  auto lut = dec_lut();
  const int nw = maxbits / 32;
  size_t nb = csw::geom_blocks(g);
  for (size_t b = 0; b < nb; b++) {
    float q[64];
    PadSource s{in + b * nw, nw};
    csw::decode_block3_pos(s, maxbits, q, lut.data(), csw::pipe_consts());
    csw::scatter_block<3>(g, out, b, q);
  }
}
// maxbits must be a multiple of 32 here (whole words per block)
void core_encode(const float* in, size_t nx, size_t ny, size_t nz, int maxbits, uint32_t* out) {
  csw::FieldGeom g = csw::make_geom(nx, ny, nz, 0, 0, 0);
  if (g.dims == 3) encode_field<3>(g, in, maxbits, out);
  else if (g.dims == 2) encode_field<2>(g, in, maxbits, out);
  else encode_field<1>(g, in, maxbits, out);
}
void core_decode(const uint32_t* in, size_t nx, size_t ny, size_t nz, int maxbits, float* out) {
  csw::FieldGeom g = csw::make_geom(nx, ny, nz, 0, 0, 0);
  if (g.dims == 3) decode_field<3>(g, in, maxbits, out);
  else if (g.dims == 2) decode_field<2>(g, in, maxbits, out);
  else decode_field<1>(g, in, maxbits, out);
}
size_t core_stream_bytes(size_t nx, size_t ny, size_t nz, unsigned maxbits) {
  return csw::stream_bytes(csw::make_geom(nx, ny, nz, 0, 0, 0), maxbits);
}
}
