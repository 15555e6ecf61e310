/*
 * s2cnn_b200 - C ABI of the B200-native spectral hot path of s2cnn.
 *
 * Every entry point takes plain pointers and sizes.  Device pointers must be float32, contiguous,
 * 16-byte aligned and live on the current CUDA device; `stream` is a cudaStream_t passed as void*
 * (NULL = the legacy default stream).  All functions return 0 on success and a non-zero status
 * otherwise, with a message available from s2c_last_error() (thread-local).  Nothing is thrown
 * across the boundary.  Except for the constant tables (built and uploaded on the first call that
 * needs a given bandwidth on a given device, and kept until s2c_clear_tables()), the library
 * allocates no device memory: scratch space is passed in by the caller (`workspace`), sized by
 * the matching *_workspace() query.  Because that first call allocates and copies synchronously,
 * warm each shape up once before capturing a CUDA graph.
 *
 * Layout conventions are the reference's: complex numbers are pairs of floats (re, im) in a
 * trailing axis of size 2; spectra carry the spectral index first,
 *   S2    : row l*l + (l+m),                         l < b, |m| <= l           (b*b rows)
 *   SO(3) : row l(4l*l-1)/3 + (l+m)(2l+1) + (l+n),   l < b, |m|,|n| <= l       (b(4b*b-1)/3 rows)
 * signals are [batch, beta, alpha(, gamma)] on the SOFT grid with 2b samples per angle.
 * `nbatch` is the product of all leading (batch, feature) dimensions.
 *
 * Each declaration cites the interface of the reference (jonkhler/s2cnn) that it replaces.
 */
#ifndef S2CNN_B200_H_
#define S2CNN_B200_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status / bookkeeping ------------------------------------------------------------------ */
const char* s2c_last_error(void);
int s2c_version(void);
/* Number of kernels this thread has launched through the library (monotonic counter). */
long s2c_launch_count(void);
/* Frees the cached tables of every device (replaces nothing in the reference; its lru_caches
 * are never cleared). */
void s2c_clear_tables(void);
/* On-disk cache of the Wigner tables: `dir` (an existing directory) turns it on, NULL or "" off;
 * unset, the environment variable S2CNN_B200_TABLE_CACHE is consulted once.  One file per (kind,
 * bandwidths, weighting), written under a temporary name and renamed into place, verified by a
 * checksum when read - safe with several processes.  Replaces the reference's cached_dirpklgz
 * decorator (s2cnn/utils/decorator.py:54-104) around its table builders.  The two counters report
 * tables read from / written to the directory by this process. */
void s2c_set_table_cache_dir(const char* dir);
long s2c_table_cache_hits(void);
long s2c_table_cache_stores(void);
/* Number of Wigner tables this process has computed from scratch so far (the host side logs a
 * message when it grows, as the reference does at s2cnn/soft/so3_fft.py:223, s2_fft.py:127). */
long s2c_tables_computed(void);
/* Per-kernel timing for benchmarks (no counterpart in the reference): between begin and end every
 * launch is bracketed by a CUDA event pair on its own stream; end() waits for them and writes one
 * text line per kernel, "<name> <launches> <total_ms>", into buf. */
void s2c_timing_begin(void);
int s2c_timing_end(char* buf, size_t buf_bytes);
/* 1 when the library was built for the GPU, 0 for the host-emulation build used by the tests. */
int s2c_is_cuda_build(void);

/* ---- host-side float64 generators (replace lie_learn calls) -------------------------------- */
/* d^l_mn(beta), (2l+1)x(2l+1) row-major, m,n = -l..l.
 * Replaces lie_learn wigner_d_matrix as called at s2cnn/soft/so3_fft.py:229-230. */
int s2c_wigner_d(int l, double beta, double* out);
/* SOFT quadrature weights, 2b values.  Replaces lie_learn S3.quadrature_weights
 * (s2cnn/soft/so3_fft.py:220, s2cnn/soft/so3_integrate.py:37). */
int s2c_quadrature_weights(int b, double* out);
/* Wigner table in the reference's own layout [2b, nspec(nl)] (float32):
 * s2cnn/soft/so3_fft.py:212-243 (_setup_so3_fft). */
int s2c_so3_wigner_table(int b, int nl, int weighted, float* out);
/* [2b, nl*nl]: s2cnn/soft/s2_fft.py:116-147 (_setup_s2_fft). */
int s2c_s2_wigner_table(int b, int nl, int weighted, float* out);
/* Fourier matrix of a kernel grid, F[n_grid][b*b][2], grid = n_grid x (beta, alpha) doubles.
 * Replaces __setup_s2_ft, s2cnn/s2_ft.py:27-50. */
int s2c_s2_ft_matrix(int b, const double* grid, int n_grid, float* F);
/* F[n_grid][nspec(b)][2], grid = n_grid x (beta, alpha, gamma).
 * Replaces __setup_so3_ft, s2cnn/so3_ft.py:27-52. */
int s2c_so3_ft_matrix(int b, const double* grid, int n_grid, float* F);

/* ---- SO(3) transforms ----------------------------------------------------------------------- */
/* Recommended scratch size (bytes) for any of the four SO(3) transforms below; any size that
 * holds at least one batch element works (the batch is processed in chunks). */
size_t s2c_so3_fft_workspace(long nbatch, int b_in, int b_out);
size_t s2c_so3_fft_workspace_min(int b_in, int b_out);

/* x [nbatch, 2b_in, 2b_in, 2b_in] real -> out [nspec(b_out), nbatch, 2].
 * Replaces so3_rfft, s2cnn/soft/so3_fft.py:64-112 (+ kernel so3fft.cu :246-350, REAL_IN). */
int s2c_so3_rfft(const float* x, float* out, long nbatch, int b_in, int b_out, int for_grad,
                 void* workspace, size_t workspace_bytes, void* stream);
/* s2c_so3_rfft of max(x, 0): the ReLU that precedes an SO3Convolution in the reference's models
 * (e.g. examples/mnist/run.py:88-93) applied while the signal is read, so the activated tensor
 * never exists in memory.  Only for 2 b_in <= 32 (single-kernel path); other sizes return
 * "unsupported". */
int s2c_so3_rfft_relu(const float* x, float* out, long nbatch, int b_in, int b_out,
                      void* workspace, size_t workspace_bytes, void* stream);
/* s2c_so3_rfft plus one by-product: sums [nbatch] = the plain sum of every signal over its (2b)^3
 * samples (read off the (m, n) = (0, 0) bins inside the kernel).  With x the gradient of a layer's
 * output this is what the gradient of the bias added at s2cnn/soft/s2_conv.py:45 / so3_conv.py:56
 * needs (summed over the batch by the caller), without another pass over the largest tensor of the
 * step.  Only for 2 b_in <= 32 (single-kernel path); other sizes return status 4 ("unsupported")
 * and write nothing. */
int s2c_so3_rfft_sums(const float* x, float* out, float* sums, long nbatch, int b_in, int b_out,
                      int for_grad, void* stream);
/* x [nbatch, 2b_in, 2b_in, 2b_in, 2] complex -> out [nspec(b_out), nbatch, 2].
 * Replaces so3_fft, s2cnn/soft/so3_fft.py:12-61. */
int s2c_so3_fft(const float* x, float* out, long nbatch, int b_in, int b_out, int for_grad,
                void* workspace, size_t workspace_bytes, void* stream);
/* x [nspec(b_in), nbatch, 2] -> out [nbatch, 2b_out, 2b_out, 2b_out] real: the real part of the
 * full complex synthesis for ANY spectrum (the reference's CPU semantics, so3_fft.py:184-199).
 * `bias` (optional, [nfeature]) is added to every sample of row z with feature z % nfeature - the
 * "+ bias" of s2cnn/soft/s2_conv.py:45 and so3_conv.py:56 fused into the last pass.
 * Replaces so3_rifft, s2cnn/soft/so3_fft.py:158-202 (+ kernel so3ifft.cu :353-443, REAL_OUT). */
int s2c_so3_rifft(const float* x, float* out, long nbatch, int b_in, int b_out, int for_grad,
                  const float* bias, int nfeature, void* workspace, size_t workspace_bytes,
                  void* stream);
/* Backward of "so3_rfft(relu(a))" with respect to a, in one kernel:
 *   out = so3_rifft(x, for_grad = 1, b_out) where act > 0, else 0
 * x [nspec(b_in), nbatch, 2] = gradient of the spectrum, act [nbatch, 2b_out, 2b_out, 2b_out] = the
 * signal the forward pass read, out of the same shape.  Only for 2 b_out <= 32 (single-kernel path);
 * other sizes return "unsupported".  Replaces the backward of SO3_fft_real (s2cnn/soft/so3_fft.py:
 * 453-456: so3_ifft(for_grad=True), real part) followed by the backward of F.relu. */
int s2c_so3_rifft_relu_grad(const float* x, const float* act, float* out, long nbatch, int b_in,
                            int b_out, void* stream);
/* so3_integrate(relu(so3_rifft(x) + bias)) without writing the signal: out [nbatch] - the tail
 * "SO3Convolution -> ReLU -> so3_integrate" of the reference's classifiers (e.g.
 * examples/mnist/run.py:88-97) in the synthesis kernel.  Only for 2 b_out <= 32 (single-kernel
 * path); other sizes return "unsupported".  Replaces so3_rifft (s2cnn/soft/so3_fft.py:158-202)
 * followed by so3_integrate (s2cnn/soft/so3_integrate.py:7-29). */
int s2c_so3_rifft_relu_integrate(const float* x, float* out, long nbatch, int b_in, int b_out,
                                 const float* bias, int nfeature, void* stream);
/* Two layers' transforms in one kernel, the signal between them never written:
 *   out = so3_rfft(relu(so3_rifft(s2_mm(xs, ys)) + bias), b_out = b_next)
 * xs [b*b, nbatch, f_in, 2], ys [b*b, f_in, f_out, 2], bias [f_out] or NULL,
 * out [nspec(b_next), nbatch, f_out, 2].  Only for 2 b <= 32 and b_next <= b; other sizes return
 * "unsupported".  Replaces the tail of S2Convolution.forward (s2cnn/soft/s2_conv.py:42-45), the ReLU
 * and the head of the next SO3Convolution.forward (s2cnn/soft/so3_conv.py:50). */
int s2c_s2_conv_relu_so3_rfft(const float* xs, const float* ys, float* out, int nbatch, int f_in,
                              int f_out, int b, int b_next, const float* bias, void* stream);
/* The same relay between two SO3Convolutions:
 *   out = so3_rfft(relu(so3_rifft(x, b_out = b_mid) + bias), b_out = b_next)
 * x [nspec(b_in), nbatch, 2], out [nspec(b_next), nbatch, 2]; bias [nfeature] or NULL as in
 * s2c_so3_rifft.  Only for 2 b_mid <= 32, b_in <= b_mid, b_next <= b_mid.  Replaces the tail of one
 * SO3Convolution.forward (s2cnn/soft/so3_conv.py:55-56), the ReLU and the head of the next (:50). */
int s2c_so3_rifft_relu_rfft(const float* x, float* out, long nbatch, int b_in, int b_mid, int b_next,
                            const float* bias, int nfeature, void* stream);
/* Same result as s2c_so3_rifft, for callers that cannot obtain device memory at call time (a
 * process whose GPU memory is wholly pre-reserved by another allocator, or a loop that must avoid
 * the device-wide synchronisation of cudaMalloc/cudaFree): no workspace argument and no device
 * allocation inside.  Scratch and tables live in two static device arrays that every GPU loading
 * the library holds until exit (32 MiB + 4 MiB).  A call whose scratch need - nbatch *
 * (K N^2 + K (2K - 1) N) * 8 bytes with N = 2 b_out and K = min(b_in, b_out), which equals
 * s2c_so3_fft_workspace_min(b_in, b_out) * nbatch when b_in <= b_out and is smaller otherwise -
 * exceeds s2c_so3_rifft_static_max_bytes(), or whose tables exceed 4 MiB, is rejected with an
 * error.  The first call on a device, and any call
 * that changes (b_in, b_out, for_grad), looks up the arrays' device addresses and uploads tables
 * synchronously: issue it before any stream capture.  All calls on a device share the arrays, so
 * calls that overlap on the GPU (other streams or threads) race; nothing has to be cleared between
 * calls.  This entry point has no counterpart in the reference. */
int s2c_so3_rifft_static(const float* x, float* out, long nbatch, int b_in, int b_out,
                         int for_grad, const float* bias, int nfeature, void* stream);
size_t s2c_so3_rifft_static_max_bytes(void);
/* The tail of S2Convolution.forward in one call (s2cnn/soft/s2_conv.py:42-45):
 *   out = so3_rifft(s2_mm(xs, ys)) + bias
 * xs [b*b, nbatch, f_in, 2], ys [b*b, f_in, f_out, 2], out [nbatch, f_out, 2b, 2b, 2b], bias [f_out]
 * or NULL.  For 2b <= 32 the product is evaluated inside the synthesis kernel and the SO(3)
 * spectrum is never written to memory; larger b run the two steps through the workspace. */
size_t s2c_s2_conv_synthesis_workspace(int nbatch, int f_out, int b);
int s2c_s2_conv_synthesis(const float* xs, const float* ys, float* out, int nbatch, int f_in,
                          int f_out, int b, const float* bias, void* workspace,
                          size_t workspace_bytes, void* stream);
/* x [nspec(b_in), nbatch, 2] -> out [nbatch, 2b_out, 2b_out, 2b_out, 2] complex.
 * Replaces so3_ifft, s2cnn/soft/so3_fft.py:115-155. */
int s2c_so3_ifft(const float* x, float* out, long nbatch, int b_in, int b_out, int for_grad,
                 void* workspace, size_t workspace_bytes, void* stream);

/* ---- S2 transforms -------------------------------------------------------------------------- */
size_t s2c_s2_fft_workspace(long nbatch, int b_in, int b_out);
/* x [nbatch, 2b_in, 2b_in(, 2)] (real when x_is_real, else complex) -> out [b_out^2, nbatch, 2];
 * requires b_out <= b_in.  Replaces s2_fft and S2_fft_real.forward,
 * s2cnn/soft/s2_fft.py:13-58,226-232 (+ kernel s2fft.cu :151-185). */
int s2c_s2_fft(const float* x, int x_is_real, float* out, long nbatch, int b_in, int b_out,
               int for_grad, void* workspace, size_t workspace_bytes, void* stream);
/* x [b_in^2, nbatch, 2] -> out [nbatch, 2b_out, 2b_out(, 2)] (real part only when out_is_real);
 * requires b_out >= b_in.  Replaces s2_ifft and S2_ifft_real.forward,
 * s2cnn/soft/s2_fft.py:61-106,239-245 (+ kernel s2ifft.cu :188-223). */
int s2c_s2_ifft(const float* x, float* out, int out_is_real, long nbatch, int b_in, int b_out,
                int for_grad, void* workspace, size_t workspace_bytes, void* stream);

/* ---- spectral products ---------------------------------------------------------------------- */
/* z[l,m,n,i,j] = sum_{p,k} x[l,m,p,i,k] conj(y[l,n,p,k,j]);  x [nspec(nl), nbatch, f_in, 2],
 * y [nspec(nl), f_in, f_out, 2], z [nspec(nl), nbatch, f_out, 2].
 * Replaces so3_mm / _cuda_SO3_mm.forward, s2cnn/so3_mm.py:8-93. */
int s2c_so3_mm(const float* x, const float* y, float* z, int nl, int nbatch, int f_in, int f_out,
               void* stream);
/* Synchronises the device and returns 0 if no tensor-core so3_mm launch has reported a barrier
 * time-out since the library was loaded, 1 if one has, -1 on a CUDA error (no counterpart in the
 * reference). */
int s2c_so3_mm_tc_status(void);
/* gx = d/dx: replaces _cuda_SO3_mm.backward (grad-x instantiation), s2cnn/so3_mm.py:108-113. */
int s2c_so3_mm_gradx(const float* gz, const float* y, float* gx, int nl, int nbatch, int f_in,
                     int f_out, void* stream);
/* gy = d/dy: replaces _cuda_SO3_mm.backward (grad-y instantiation), s2cnn/so3_mm.py:115-120. */
int s2c_so3_mm_grady(const float* gz, const float* x, float* gy, int nl, int nbatch, int f_in,
                     int f_out, void* stream);
/* z[l,m,n,i,j] = sum_k x[l,m,i,k] conj(y[l,n,k,j]);  x [nl^2, nbatch, f_in, 2],
 * y [nl^2, f_in, f_out, 2], z [nspec(nl), nbatch, f_out, 2].
 * Replaces s2_mm / _cuda_s2_mm, s2cnn/s2_mm.py:10-28,104-137 (+ kernel s2mm.cu :140-198). */
int s2c_s2_mm(const float* x, const float* y, float* z, int nl, int nbatch, int f_in, int f_out,
              void* stream);
/* Replaces _cuda_S2_mm.backward grad-x, s2cnn/s2_mm.py:85-92 (+ s2mm_gradx.cu :201-255). */
int s2c_s2_mm_gradx(const float* gz, const float* y, float* gx, int nl, int nbatch, int f_in,
                    int f_out, void* stream);
/* Replaces _cuda_S2_mm.backward grad-y, s2cnn/s2_mm.py:94-99 (+ s2mm_grady.cu :258-312). */
int s2c_s2_mm_grady(const float* gz, const float* x, float* gy, int nl, int nbatch, int f_in,
                    int f_out, void* stream);

/* ---- kernel-grid -> spectrum transforms ----------------------------------------------------- */
/* out[s, f, :] = sum_a x[f, a] F[a, s, :];  x [nf, n_grid], F [n_grid, nspec, 2] (device),
 * out [nspec, nf, 2].  Replaces the einsum of s2_rft / so3_rft, s2cnn/s2_ft.py:22,
 * s2cnn/so3_ft.py:22. */
int s2c_rft_forward(const float* x, const float* F, float* out, int nf, int n_grid, int nspec,
                    void* stream);
/* The same product on the tensor cores (tcgen05, 3xTF32), given the TRANSPOSED matrix
 * Ft [nspec, 2, n_grid] (the caller keeps it beside F); needs an even n_grid and the CUDA build,
 * other cases return "unsupported" (use s2c_rft_forward). */
int s2c_rft_forward_t(const float* x, const float* Ft, float* out, int nf, int n_grid, int nspec,
                      void* stream);
/* gx[f, a] = sum_{s,c} g[s, f, c] F[a, s, c]: the autograd transpose of the einsum above (on the
 * tensor cores when n_grid is even). */
int s2c_rft_backward(const float* g, const float* F, float* gx, int nf, int n_grid, int nspec,
                     void* stream);

/* ---- integration ---------------------------------------------------------------------------- */
/* out[z] = sum_beta w_beta sum_{alpha,gamma} x[z, beta, alpha, gamma]; x [n, 2b, 2b, 2b].
 * With relu != 0 the integrand is max(x, 0) (activation fused into the read).
 * Replaces so3_integrate, s2cnn/soft/so3_integrate.py:7-29. */
int s2c_so3_integrate(const float* x, float* out, long n, int b, int relu, void* stream);
/* gx[z, beta, :, :] = g[z] w_beta (masked by x > 0 when relu != 0; x may be NULL otherwise). */
int s2c_so3_integrate_backward(const float* g, const float* x, float* gx, long n, int b, int relu,
                               void* stream);

/* ---- rotation of a signal on SO(3) ------------------------------------------------------------ */
/* HOST generator: out = concatenation over l < b of U^l[m, n] = exp(i m alpha) d^l_mn(beta)
 * exp(i n gamma), interleaved complex floats, b(4b^2-1)/3 entries.  Replaces the lie_learn
 * wigner_D_matrix call of __setup_so3_rotation, s2cnn/soft/so3_rotation.py:51-62. */
int s2c_so3_rotation_matrices(int b, double alpha, double beta, double gamma, float* out);
/* DEVICE: z[l,m,n,c] = sum_k conj(U^l[m,k]) x[l,k,n,c]   (adjoint == 0), or the transposed product
 * gx[l,k,n,c] = sum_m U^l[m,k] gz[l,m,n,c]               (adjoint != 0), for spectra
 * [b(4b^2-1)/3, nbatch, 2].  Replaces the per-degree complex_mm loop of so3_rotation,
 * s2cnn/soft/so3_rotation.py:22-41 (and, with adjoint, its autograd). */
int s2c_so3_rotate_spectrum(const float* U, const float* x, float* z, int b, long nbatch,
                            int adjoint, void* stream);

/* ---- data preparation of the 3-D shape model --------------------------------------------------- */
/* Ray-cast projection of a triangle mesh onto sphere grid points: verts [nv][3] float32, faces
 * [nf][3] int32 (vertex indices, not range-checked), grid [nr][3] ray origins (direction = towards
 * the origin), all on the device; out [3][nr] = distance to the first hit (1 if none), n . p and
 * |n x p| with n the hit triangle's unit normal and p the normalised origin (0 if none).  Replaces
 * render_model, examples/shrec17/dataset.py:53-95 (trimesh / pyembree ray casting on the host). */
int s2c_project_on_sphere(const float* verts, int nv, const int* faces, int nf, const float* grid,
                          int nr, float* out, void* stream);

/* ---- test hooks (not part of the drop-in surface; no counterpart in the reference) ------------ */
/* Path selection for the test-suite, so that every kernel variant can be compared with the oracle
 * at the same sizes.  The switches are process-wide atomics read once per call by the dispatcher;
 * an application has no reason to touch them.
 *   s2c_debug_force_general_path(level): 1 routes small bandwidths (2b <= 32) through the general
 *     kernels instead of the single-kernel path; 2 additionally replaces the plane kernels of
 *     2b = 64 / 128 (both row transforms of a (z, beta) plane in one kernel) by the three separate
 *     passes every other size uses; 0 restores the defaults.
 *   s2c_debug_plane_chunk(signals): signals per chunk of the large-bandwidth path (1 .. 8); 0
 *     restores the default (8, or what the workspace holds). */
void s2c_debug_force_general_path(int level);
void s2c_debug_plane_chunk(int signals);

#ifdef __cplusplus
}
#endif
#endif /* S2CNN_B200_H_ */
