"""Projection of triangle meshes onto the sphere grid: the data preparation in front of the 3-D
shape model of the reference's examples (examples/shrec17/dataset.py:14-182).

``make_sgrid`` and ``rotmat`` restate the reference's helpers (the SOFT grid comes from the formula
lie_learn's ``S2.meshgrid(b, 'SOFT')`` implements: theta_j = pi (2j + 1) / (4b), phi_k = pi k / b).
``render_model`` runs the ray casting - trimesh / pyembree on the host in the reference - as a CUDA
kernel (``s2c_project_on_sphere``).  ``ProjectOnSphere`` assembles the six input channels of the
model (three from the mesh, three from its convex hull) with the reference's normalisation
constants.  Meshes are given as (vertices [nv, 3], faces [nf, 3]); loading and cleaning mesh files is
the caller's business (the reference uses trimesh for that).
"""
import numpy as np
import torch

from .ops import cuda_ops


def rotmat(a, b, c, hom_coord=False):
    """ZYZ Euler rotation matrix (examples/shrec17/dataset.py:14-37), 3x3 or homogeneous 4x4."""
    def z(t):
        return np.array([[np.cos(t), np.sin(t), 0, 0], [-np.sin(t), np.cos(t), 0, 0],
                         [0, 0, 1, 0], [0, 0, 0, 1]])

    def y(t):
        return np.array([[np.cos(t), 0, np.sin(t), 0], [0, 1, 0, 0],
                         [-np.sin(t), 0, np.cos(t), 0], [0, 0, 0, 1]])

    r = z(a).dot(y(b)).dot(z(c))
    return r if hom_coord else r[:3, :3]


def make_sgrid(b, alpha=0.0, beta=0.0, gamma=0.0):
    """The (2b)^2 points of the SOFT grid on the unit sphere, beta-major, rotated by the ZYZ Euler
    angles: float64 [4 b^2, 3] (examples/shrec17/dataset.py:40-50)."""
    theta = np.pi * (2 * np.arange(2 * b) + 1) / (4 * b)
    phi = np.pi * np.arange(2 * b) / b
    t, p = np.meshgrid(theta, phi, indexing="ij")
    pts = np.stack((np.sin(t) * np.cos(p), np.sin(t) * np.sin(p), np.cos(t)), axis=-1).reshape(-1, 3)
    return np.einsum("ij,nj->ni", rotmat(alpha, beta, gamma), pts)


def render_model(vertices, faces, sgrid, device="cuda:0"):
    """Three spherical images [3, n_points] of a mesh seen from the grid points (rays towards the
    origin, first hit): distance (1 where nothing is hit), normal . ray and |normal x ray| (0 where
    nothing).  Same channels as examples/shrec17/dataset.py:53-95."""
    ops = cuda_ops()
    v = torch.as_tensor(np.ascontiguousarray(vertices, dtype=np.float32)).to(device)
    f = torch.as_tensor(np.ascontiguousarray(faces, dtype=np.int32)).to(device)
    g = torch.as_tensor(np.ascontiguousarray(sgrid, dtype=np.float32)).to(device)
    return ops.project_on_sphere(v, f, g)


class ProjectOnSphere:
    """mesh -> float32 tensor [6, 2b, 2b] on the device: the mesh's three channels, then its convex
    hull's, shifted and scaled by the reference's per-channel constants
    (examples/shrec17/dataset.py:146-182).  The hull comes from scipy (qhull) on the host; if qhull
    fails the mesh itself is used, as in the reference."""

    SHIFT = (0.75, 0.59, 0.54, 0.52, 0.80, 0.51)
    SCALE = (0.26, 0.50, 0.29, 0.19, 0.18, 0.25)

    def __init__(self, bandwidth, device="cuda:0"):
        self.bandwidth = bandwidth
        self.device = device
        self.sgrid = make_sgrid(bandwidth)

    @staticmethod
    def convex_hull(vertices):
        from scipy.spatial import ConvexHull
        v = np.asarray(vertices, dtype=np.float64)
        hull = ConvexHull(v)
        faces = hull.simplices.copy()
        # orient every triangle outwards (qhull does not order the vertices of a simplex)
        centre = v[hull.vertices].mean(axis=0)
        a, b, c = v[faces[:, 0]], v[faces[:, 1]], v[faces[:, 2]]
        flip = np.einsum("ij,ij->i", np.cross(b - a, c - a), a - centre) < 0
        faces[flip] = faces[flip][:, ::-1]
        return v, faces

    def __call__(self, vertices, faces):
        n = 2 * self.bandwidth
        im = render_model(vertices, faces, self.sgrid, self.device)
        try:
            hv, hf = self.convex_hull(vertices)
        except Exception:  # noqa: BLE001  (qhull errors)
            hv, hf = vertices, faces
        hull_im = render_model(hv, hf, self.sgrid, self.device)
        out = torch.cat((im, hull_im), dim=0)
        shift = torch.tensor(self.SHIFT, device=out.device).view(6, 1)
        scale = torch.tensor(self.SCALE, device=out.device).view(6, 1)
        return ((out - shift) / scale).view(6, n, n)

    def __repr__(self):
        return "%s(bandwidth=%d)" % (type(self).__name__, self.bandwidth)
