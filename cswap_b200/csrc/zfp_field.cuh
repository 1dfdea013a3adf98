// Field geometry of the ZFP codec: block index -> origin, strided gather with
// replicate padding of partial blocks, scatter, and stream sizing.
// Follows CSWAP+/zfp/encode3.cuh:12-47,78-105, encode2.cuh, encode1.cuh,
// encode.cuh:17-38 (pad_block), decode3.cuh:10-39 and shared.h:39-84.
// Plain scalar code, shared by the generic CUDA kernels and host-side tests.
#pragma once
#include <cstddef>
#include <cstdint>

#include "zfp_core.cuh"

namespace csw {

struct FieldGeom {
  uint32_t nx, ny, nz;     // extents; ny = 0 / nz = 0 for lower-dimensional fields
  int64_t sx, sy, sz;      // element strides
  uint32_t bx, by, bz;     // blocks per axis
  int dims;
};

inline FieldGeom make_geom(size_t nx, size_t ny, size_t nz, int64_t sx, int64_t sy, int64_t sz) {
  FieldGeom g;
  g.nx = (uint32_t)nx; g.ny = (uint32_t)ny; g.nz = (uint32_t)nz;
  g.dims = nz ? 3 : ny ? 2 : 1;
  // zero strides mean contiguous (cuZFP.cu:372-375)
  g.sx = sx ? sx : 1;
  g.sy = sy ? sy : (int64_t)nx;
  g.sz = sz ? sz : (int64_t)nx * (int64_t)(ny ? ny : 1);
  g.bx = (g.nx + 3) / 4;
  g.by = g.dims >= 2 ? (g.ny + 3) / 4 : 1;
  g.bz = g.dims >= 3 ? (g.nz + 3) / 4 : 1;
  return g;
}

inline size_t geom_blocks(const FieldGeom& g) { return (size_t)g.bx * g.by * g.bz; }

// Bytes of whole 64-bit words covering every (padded) block.  The reference's
// own counts (shared.h:39-84) truncate for 3-D and count unpadded values for
// 1-D/2-D; they agree with this whenever maxbits % 64 == 0 and no block is
// partial.
inline size_t stream_bytes(const FieldGeom& g, unsigned maxbits) {
  return (geom_blocks(g) * maxbits + 63) / 64 * 8;
}

// encode.cuh:17-38: n valid values along a line of stride s -> 4 values
CSW_HD void pad_line(float* p, uint32_t n, int s) {
  if (n == 0) p[0] = 0.0f;
  if (n <= 1) p[s] = p[0];
  if (n <= 2) p[2 * s] = p[s];
  if (n <= 3) p[3 * s] = p[0];
}

template <int DIMS>
CSW_HD void gather_block(const FieldGeom& g, const float* in, size_t b, float (&q)[1 << (2 * DIMS)]) {
  const uint32_t x0 = (uint32_t)(b % g.bx) * 4;
  const uint32_t y0 = DIMS >= 2 ? (uint32_t)((b / g.bx) % g.by) * 4 : 0;
  const uint32_t z0 = DIMS >= 3 ? (uint32_t)(b / ((size_t)g.bx * g.by)) * 4 : 0;
  const uint32_t vx = g.nx - x0 < 4 ? g.nx - x0 : 4;
  const uint32_t vy = DIMS >= 2 ? (g.ny - y0 < 4 ? g.ny - y0 : 4) : 1;
  const uint32_t vz = DIMS >= 3 ? (g.nz - z0 < 4 ? g.nz - z0 : 4) : 1;
  const float* base = in + (int64_t)x0 * g.sx + (int64_t)y0 * g.sy + (int64_t)z0 * g.sz;
  for (uint32_t z = 0; z < vz; z++) {
    for (uint32_t y = 0; y < vy; y++) {
      for (uint32_t x = 0; x < vx; x++)
        q[16 * z + 4 * y + x] = base[(int64_t)x * g.sx + (int64_t)y * g.sy + (int64_t)z * g.sz];
      if (vx < 4) pad_line(&q[16 * z + 4 * y], vx, 1);
    }
    if constexpr (DIMS >= 2) {
      if (vy < 4)
        for (int x = 0; x < 4; x++) pad_line(&q[16 * z + x], vy, 4);
    }
  }
  if constexpr (DIMS >= 3) {
    if (vz < 4)
      for (int i = 0; i < 16; i++) pad_line(&q[i], vz, 16);
  }
}

template <int DIMS>
CSW_HD void scatter_block(const FieldGeom& g, float* out, size_t b, const float (&q)[1 << (2 * DIMS)]) {
  const uint32_t x0 = (uint32_t)(b % g.bx) * 4;
  const uint32_t y0 = DIMS >= 2 ? (uint32_t)((b / g.bx) % g.by) * 4 : 0;
  const uint32_t z0 = DIMS >= 3 ? (uint32_t)(b / ((size_t)g.bx * g.by)) * 4 : 0;
  const uint32_t vx = g.nx - x0 < 4 ? g.nx - x0 : 4;
  const uint32_t vy = DIMS >= 2 ? (g.ny - y0 < 4 ? g.ny - y0 : 4) : 1;
  const uint32_t vz = DIMS >= 3 ? (g.nz - z0 < 4 ? g.nz - z0 : 4) : 1;
  float* base = out + (int64_t)x0 * g.sx + (int64_t)y0 * g.sy + (int64_t)z0 * g.sz;
  for (uint32_t z = 0; z < vz; z++)
    for (uint32_t y = 0; y < vy; y++)
      for (uint32_t x = 0; x < vx; x++)
        base[(int64_t)x * g.sx + (int64_t)y * g.sy + (int64_t)z * g.sz] = q[16 * z + 4 * y + x];
}

}  // namespace csw
