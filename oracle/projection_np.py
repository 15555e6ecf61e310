"""Test infrastructure: float64 numpy restatement of the reference's spherical projection of a mesh
(examples/shrec17/dataset.py:53-95, render_model).  The reference hands the ray casting to trimesh
(``mesh.ray.intersects_id(..., multiple_hits=False)``), which is absent here; what is restated is
the published algorithm behind that call - first intersection of each ray with the triangle soup,
Moeller-Trumbore test - and the three channels the reference builds from the hits.  Parity of this
oracle is unpinned (no trimesh to compare with); it is pinned only to analytic cases in the tests
(a sphere-like mesh seen from its centre direction, rays that miss).
"""
import numpy as np


def render_model(vertices, faces, sgrid):
    v = np.asarray(vertices, dtype=np.float64)
    f = np.asarray(faces, dtype=np.int64)
    o = np.asarray(sgrid, dtype=np.float64)           # ray origins; directions are -o  (:57-58)
    d = -o
    v0 = v[f[:, 0]]
    e1 = v[f[:, 1]] - v0
    e2 = v[f[:, 2]] - v0
    normals = np.cross(e1, e2)
    nn = np.linalg.norm(normals, axis=1, keepdims=True)
    normals = normals / np.where(nn > 0, nn, 1.0)     # trimesh face_normals are unit vectors (:70-71)
    n_rays = o.shape[0]
    best_t = np.full(n_rays, np.inf)
    best_f = np.full(n_rays, -1)
    for j in range(f.shape[0]):                        # one triangle at a time keeps memory small
        p = np.cross(d, e2[j])
        det = p @ e1[j]
        ok = np.abs(det) > 1e-12
        idet = np.where(ok, 1.0 / np.where(ok, det, 1.0), 0.0)
        s = o - v0[j]
        u = np.einsum("ij,ij->i", s, p) * idet
        q = np.cross(s, e1[j])
        w = np.einsum("ij,ij->i", d, q) * idet
        t = (q @ e2[j]) * idet
        hit = ok & (u >= 0) & (u <= 1) & (w >= 0) & (u + w <= 1) & (t > 0) & (t < best_t)
        best_t = np.where(hit, t, best_t)
        best_f = np.where(hit, j, best_f)
    hit = best_f >= 0
    g = o / np.linalg.norm(o, axis=1, keepdims=True)   # grid_hits_normalized (:63)
    dist = np.ones(n_rays)                             # :74
    dist[hit] = best_t[hit] * np.linalg.norm(o[hit], axis=1)   # |origin - hit point| (:66)
    n = normals[np.where(hit, best_f, 0)]
    ndot = np.where(hit, np.einsum("ij,ij->i", n, g), 0.0)      # :81-83
    wedge = np.where(hit, np.linalg.norm(np.cross(n, g), axis=1), 0.0)   # :85-89
    return np.stack((dist, ndot, wedge), axis=0)       # :93
