"""Test infrastructure (oracle side): Wigner-d / Wigner-D samples and SOFT quadrature
weights in float64 numpy.

The reference obtains these three functions from the third-party package ``lie_learn``
(named in the reference's README.md:15, no version pinned anywhere in the reference, not
vendored).  Call sites in the reference:

* ``wigner_d_matrix(l, beta, field='complex', normalization='quantum', order='centered',
  condon_shortley='cs')`` - s2cnn/soft/so3_fft.py:214,229-230, s2cnn/soft/s2_fft.py:118,134-135
* ``wigner_D_matrix(l, alpha, beta, gamma, ...same kwargs...)`` - s2cnn/s2_ft.py:29,39-40,
  s2cnn/so3_ft.py:29,41-42, s2cnn/soft/so3_rotation.py:53-56
* ``S3.quadrature_weights(b)`` - s2cnn/soft/so3_fft.py:215,220, s2cnn/soft/s2_fft.py:119,124,
  s2cnn/soft/so3_integrate.py:35-37, tests/so3_fft.py:15-18

This file restates the published mathematics (it is not derived from lie_learn's source):

* ``d^l(beta) = exp(-i beta J_y)`` in the |l,m> basis ordered m = -l..l ("centered"), with
  ``J_+ |l,m> = sqrt(l(l+1) - m(m+1)) |l,m+1>``; the matrix is real.  Known answers:
  ``d^l(0) = I``, ``d^1_{0,0} = cos(beta)``, ``d^1_{1,0} = -sin(beta)/sqrt(2)``.
* ``D^l_mn(alpha,beta,gamma) = exp(i m alpha) d^l_mn(beta) exp(i n gamma)`` - the phase
  convention the reference states at s2cnn/soft/so3_rotation.py:58 and that its own test
  tests/so3_fft.py:8-22 pins (the opposite phase fails that test).
* Driscoll-Healy / SOFT weights on beta_j = pi (2j+1)/(4b), scaled so that
  ``sum_j w_j = 1/(2b)^2`` which is what the reference's round-trip tests
  (tests/so3_fft.py:34-91) and ``so3_integrate(ones) == 1`` require.

PARITY STATUS: "parity unpinned" for the one convention the reference's tests do not fix:
the transposition sign d^l_mn <-> d^l_nm = (-1)^(m-n) d^l_mn.  Both choices pass every test
in the reference and give identical layer outputs (the change is a diagonal similarity that
cancels through fft -> mm -> ifft); intermediate spectra differ by (-1)^(m-n).

The evaluation method here (Hermitian eigendecomposition of J_y) is deliberately different
from the three-term recurrence in l used by the library's C++ table generator, so the two
cross-check each other.
"""
from functools import lru_cache

import numpy as np


@lru_cache(maxsize=None)
def _jy_eig(l):
    """Eigen-decomposition J_y = V diag(mu) V^H for angular momentum l."""
    dim = 2 * l + 1
    m = np.arange(-l, l)  # m -> m+1
    c = np.sqrt(l * (l + 1) - m * (m + 1.0))
    jp = np.zeros((dim, dim), dtype=np.complex128)
    jp[np.arange(1, dim), np.arange(0, dim - 1)] = c  # <m+1| J+ |m>
    jy = (jp - jp.conj().T) / (2.0j)
    mu, v = np.linalg.eigh(jy)
    # eigenvalues are exactly the integers -l..l; snapping them removes the O(eps*l) error
    mu = np.rint(mu)
    return mu, v


def wigner_d_matrix(l, beta, field='complex', normalization='quantum', order='centered',
                    condon_shortley='cs'):
    """Real (2l+1)x(2l+1) matrix d^l_mn(beta), rows m and columns n ordered -l..l.

    Returns a fresh writable float64 array (the reference scales it in place,
    s2cnn/soft/so3_fft.py:233-236).
    """
    assert field == 'complex' and normalization == 'quantum'
    assert order == 'centered' and condon_shortley == 'cs'
    mu, v = _jy_eig(int(l))
    d = (v * np.exp(-1j * float(beta) * mu)[None, :]) @ v.conj().T
    return np.ascontiguousarray(d.real)


def wigner_D_matrix(l, alpha, beta, gamma, field='complex', normalization='quantum',
                    order='centered', condon_shortley='cs'):
    """Complex D^l_mn = exp(i m alpha) d^l_mn(beta) exp(i n gamma)."""
    d = wigner_d_matrix(l, beta, field, normalization, order, condon_shortley)
    m = np.arange(-l, l + 1)
    return np.exp(1j * m * alpha)[:, None] * d * np.exp(1j * m * gamma)[None, :]


def quadrature_weights(b):
    """SOFT beta-quadrature weights, length 2b, sum = 1/(2b)^2."""
    j = np.arange(2 * b)
    k = np.arange(b)
    theta = np.pi * (2 * j + 1) / (4.0 * b)
    s = (np.sin(theta[:, None] * (2 * k[None, :] + 1)) / (2 * k[None, :] + 1)).sum(axis=1)
    w = (2.0 / b) * np.sin(theta) * s
    return w / (2.0 * (2 * b) ** 2)


def soft_betas(b):
    """beta_j = pi (2j+1)/(4b)  (s2cnn/soft/so3_fft.py:219)."""
    return (np.arange(2 * b) + 0.5) / (2 * b) * np.pi
