// Projection of a triangle mesh onto the sphere grid by ray casting: the data preparation in
// front of the first layer of the reference's 3-D shape model (examples/shrec17/dataset.py:53-95,
// render_model): one ray per grid point p of the unit sphere, from p towards the origin; the first
// triangle it meets gives three channels
//   0: distance from p to the hit point                 (1 where the ray meets nothing)
//   1: n . p   with n the unit normal of the triangle   (0 where nothing)
//   2: |n x p|                                          (0 where nothing)
// The reference delegates the intersection to trimesh / pyembree on the host; here every ray tests
// every triangle (Moeller-Trumbore, float32), triangles staged through shared memory in tiles, one
// thread per ray.  With a few thousand triangles and (2b)^2 = 16384 rays this is tens of millions of
// tests - microseconds on a GPU - so no acceleration structure is built.
#pragma once

#include "backend.h"

namespace s2c {

constexpr int kProjThreads = 128;
constexpr int kProjTile = 256;      // triangles per shared-memory tile

struct ProjectParams {
  const float* verts;   // [nv][3]
  const int* faces;     // [nf][3]
  const float* grid;    // [nr][3] ray origins on the unit sphere; direction = -origin
  float* out;           // [3][nr]
  int nv, nf, nr;
};

S2C_KERNEL(project_on_sphere, ProjectParams) {
  // per triangle: v0, e1 = v1 - v0, e2 = v2 - v0, unit normal  (12 floats)
  float* tri = reinterpret_cast<float*>(smem);
  const int ray = ctx.bid * ctx.nthr + ctx.tid;
  float ox = 0.f, oy = 0.f, oz = 0.f;
  if (ray < p.nr) { ox = p.grid[3 * ray]; oy = p.grid[3 * ray + 1]; oz = p.grid[3 * ray + 2]; }
  const float dx = -ox, dy = -oy, dz = -oz;
  float best_t = 3.0e38f, best_nx = 0.f, best_ny = 0.f, best_nz = 0.f;
  for (int f0 = 0; f0 < p.nf; f0 += kProjTile) {
    const int cnt = (p.nf - f0) < kProjTile ? (p.nf - f0) : kProjTile;
    ctx.sync();
    for (int i = ctx.tid; i < cnt; i += ctx.nthr) {
      const int* f = p.faces + 3 * (f0 + i);
      const float* a = p.verts + 3 * f[0];
      const float* b = p.verts + 3 * f[1];
      const float* c = p.verts + 3 * f[2];
      const float e1x = b[0] - a[0], e1y = b[1] - a[1], e1z = b[2] - a[2];
      const float e2x = c[0] - a[0], e2y = c[1] - a[1], e2z = c[2] - a[2];
      float nx = e1y * e2z - e1z * e2y, ny = e1z * e2x - e1x * e2z, nz = e1x * e2y - e1y * e2x;
      const float nn = sqrtf(nx * nx + ny * ny + nz * nz);
      const float inv = nn > 0.f ? 1.f / nn : 0.f;
      float* t = tri + 12 * i;
      t[0] = a[0]; t[1] = a[1]; t[2] = a[2];
      t[3] = e1x; t[4] = e1y; t[5] = e1z;
      t[6] = e2x; t[7] = e2y; t[8] = e2z;
      t[9] = nx * inv; t[10] = ny * inv; t[11] = nz * inv;
    }
    ctx.sync();
    if (ray < p.nr) {
      for (int i = 0; i < cnt; ++i) {
        const float* t = tri + 12 * i;
        // Moeller-Trumbore
        const float px = dy * t[8] - dz * t[7], py = dz * t[6] - dx * t[8], pz = dx * t[7] - dy * t[6];
        const float det = t[3] * px + t[4] * py + t[5] * pz;
        if (fabsf(det) < 1e-12f) continue;                       // ray parallel to the triangle
        const float idet = 1.f / det;
        const float sx = ox - t[0], sy = oy - t[1], sz = oz - t[2];
        const float u = (sx * px + sy * py + sz * pz) * idet;
        if (u < 0.f || u > 1.f) continue;
        const float qx = sy * t[5] - sz * t[4], qy = sz * t[3] - sx * t[5], qz = sx * t[4] - sy * t[3];
        const float v = (dx * qx + dy * qy + dz * qz) * idet;
        if (v < 0.f || u + v > 1.f) continue;
        const float tt = (t[6] * qx + t[7] * qy + t[8] * qz) * idet;
        if (tt > 0.f && tt < best_t) { best_t = tt; best_nx = t[9]; best_ny = t[10]; best_nz = t[11]; }
      }
    }
  }
  if (ray >= p.nr) return;
  float dist = 1.f, ndot = 0.f, wedge = 0.f;
  if (best_t < 3.0e38f) {
    // |d| = |p| (1 for a point of the unit sphere): distance along the ray = t |p|
    const float on = sqrtf(ox * ox + oy * oy + oz * oz);
    dist = best_t * on;
    const float gx = ox / on, gy = oy / on, gz = oz / on;
    ndot = best_nx * gx + best_ny * gy + best_nz * gz;
    const float wx = best_nx * gy - best_ny * gx, wy = best_nx * gz - best_nz * gx,
                wz = best_ny * gz - best_nz * gy;
    wedge = sqrtf(wx * wx + wy * wy + wz * wz);
  }
  p.out[ray] = dist;
  p.out[p.nr + ray] = ndot;
  p.out[2 * p.nr + ray] = wedge;
}

}  // namespace s2c
