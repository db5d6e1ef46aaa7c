/*
 * b200proj.h -- C ABI of the B200 (sm_100a) Fourier-slice operators.
 *
 * One entry point per raw operator of warpem/torch-projectors
 * (schemas: csrc/torch_projectors.cpp:23-36 of the reference).  Each entry point replaces
 * the reference's CUDA host wrapper + kernel for that operator and is what a binding layer
 * (the reference's TORCH_LIBRARY_IMPL(torch_projectors, CUDA, ...) block,
 * csrc/torch_projectors.cpp:82-95) would call.
 *
 * Conventions
 *  - No torch types: raw DEVICE pointers, explicit sizes, a CUDA stream handle
 *    (cudaStream_t passed as void*; NULL = the legacy default stream).
 *  - All tensors are contiguous, PyTorch rfft layout (origin at index 0, last axis holds the
 *    non-negative x frequencies).  Complex tensors are interleaved float pairs (complex64).
 *        rec    [B, (R,) R, Rh]  complex   Rh = R/2 + 1
 *        proj   [B, P, N, Nh]    complex   Nh = N/2 + 1
 *        rot    [B_rot, P, dim, dim] float (dim = 2 or 3), applied as given
 *        shifts [B_shift, P, 2]  float     ([..,0] pairs with rows, [..,1] with columns)
 *    B_rot and B_shift are 1 (shared by all batch items) or B.  shifts may be NULL
 *    (then B_shift is ignored).
 *  - interpolation: B200PROJ_LINEAR or B200PROJ_CUBIC (Catmull-Rom, a = -0.5).
 *  - fourier_radius_cutoff is in projection frequency units; pixels with
 *    kr*kr + kc*kc > cutoff*cutoff are excluded.  Pass N/2.0 for the reference's default.
 *  - Calls are asynchronous on the given stream, allocate nothing and never synchronise.
 *    The device of the pointers must be current.  One exception: the FIRST call of
 *    b200proj_backproject_2d_to_3d_forw_noalloc on a device looks up its built-in scratch, which
 *    may load the library's device code and so block and reserve device memory (see there).
 *  - Return value: B200PROJ_OK or a negative error code; b200proj_last_error() gives the
 *    message of the calling thread's last failure.  Argument errors are detected before
 *    anything is launched.
 *  - Outputs that are accumulated with atomics are zero-filled by the entry point itself
 *    (cudaMemsetAsync on the stream) unless stated otherwise.
 */
#ifndef B200PROJ_H
#define B200PROJ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200PROJ_LINEAR 0
#define B200PROJ_CUBIC 1

#define B200PROJ_OK 0
#define B200PROJ_ERR_ARGUMENT (-1)   /* bad size / flag / NULL pointer */
#define B200PROJ_ERR_LIMIT (-2)      /* size beyond what the kernels index */
#define B200PROJ_ERR_CUDA (-3)       /* a CUDA runtime call failed */

/* Library version (major*10000 + minor*100 + patch). */
int b200proj_version(void);

/* Hash of the sources (this header and the kernel files) the library was built from, as the
 * build script passed it in; "" for a build that did not.  A binding compares it with the hash
 * of the sources it was written against and refuses a library built from other ones. */
const char* b200proj_source_stamp(void);

/* Message of the calling thread's last failing call ("" if none). */
const char* b200proj_last_error(void);

/* Volume box a back-projection of N-pixel projections produces: ceil(N*oversampling),
 * rounded up to even.
 * replaces: csrc/cuda/3d/backprojection_2d_to_3d_kernels.cu:1039-1041 */
int64_t b200proj_rec_boxsize(int64_t N, double oversampling);

/* Test hook (host only, launches nothing): the result of one of the kernels' index helpers, which
 * are compiled for host and device from the same source, for a signed voxel coordinate.
 * which: 0 gather column (linear), 1 gather column (cubic), 2 gather row/plane (linear),
 * 3 gather row/plane (cubic), 4 scatter column, 5 scatter row/plane.  Gathers clamp (result is
 * always a valid index), scatters return -1 for a dropped tap.  For the column helpers
 * *mirrored_out tells whether the Friedel mate is addressed; the row/plane helpers take that flag
 * as mirrored_in.  Exists so that a CPU test can feed INT_MIN / INT_MAX (what a sample position
 * beyond +-2^31 saturates to) without running such poses on a GPU.
 * No counterpart in the reference (its CPU code indexes in int64, csrc/cpu/common/fftw_sampling.h:96-137). */
int b200proj_debug_index(int which, int R, int coordinate, int mirrored_in, int* mirrored_out);

/* ---- forward projection (gather) -------------------------------------------------------
 * out[b,p,i,j] = interp(rec[b], R_p * os * (j, freq(i)[, 0])) * exp(-2 pi i k.s / N);
 * every stored pixel is written (0 outside the cutoff), so `out` needs no pre-fill.
 * replaces: project_2d_forw_cuda       csrc/cuda/2d/projection_2d_kernels.cu:633-757
 *           project_3d_to_2d_forw_cuda csrc/cuda/3d/projection_3d_to_2d_kernels.cu:814-1015 */
int b200proj_project_2d_forw(const float* rec, int64_t B, int64_t R,
                             const float* rot, int64_t B_rot,
                             const float* shifts, int64_t B_shift,
                             int64_t P, int64_t N, int interpolation, double oversampling,
                             double fourier_radius_cutoff, float* out, void* stream);
int b200proj_project_3d_to_2d_forw(const float* rec, int64_t B, int64_t R,
                                   const float* rot, int64_t B_rot,
                                   const float* shifts, int64_t B_shift,
                                   int64_t P, int64_t N, int interpolation, double oversampling,
                                   double fourier_radius_cutoff, float* out,
                                   const int32_t* pose_order, void* stream);

/* ---- forward projection with packed output ------------------------------------------------
 * No counterpart in the reference.  For callers that move the projections off the device: only
 * the pixels inside the cutoff are produced, side by side, out_packed [B, P, pack_count] complex
 * (at cutoff N/2 that is 78 % of the stored pixels), so the zeros outside the cutoff never cross
 * PCIe.  b200proj_cutoff_pack_index (host only, launches nothing) fills index [N * Nh] with the
 * position of every pixel among the packed ones (-1 outside the cutoff), using the kernels' own
 * cutoff test, and returns their number (index may be NULL to get the count alone; -1 on bad
 * arguments).  The caller copies that table to the device once and passes it as pack_index; to
 * unpack, scatter out_packed[.., index[q]] to pixel q.  float only. */
int64_t b200proj_cutoff_pack_index(int64_t N, double fourier_radius_cutoff, int32_t* index);
int b200proj_project_3d_to_2d_forw_packed(const float* rec, int64_t B, int64_t R,
                                          const float* rot, int64_t B_rot,
                                          const float* shifts, int64_t B_shift,
                                          int64_t P, int64_t N, int interpolation, double oversampling,
                                          double fourier_radius_cutoff, float* out_packed,
                                          const int32_t* pack_index, int64_t pack_count,
                                          const int32_t* pose_order, void* stream);

/* ---- processing order of the slices (3D operators that read a volume) -------------------
 * No counterpart in the reference.  The three volume-reading 3D entry points
 * (project_3d_to_2d_forw, project_3d_to_2d_back, backproject_2d_to_3d_back) take an optional
 * `pose_order`: int32 [B*P] on the device, a permutation of the slice indices b*P + p that
 * keeps every batch item's slices inside its own range [b*P, (b+1)*P); block k of the launch
 * then handles slice pose_order[k].  Outputs stay where they belong (slice
 * b*P + p is written at index b*P + p) and their values do not depend on the order; only the
 * set of slices in flight at one time changes.  NULL = natural order.  An entry outside its
 * batch item's range makes its blocks idle (that slice is then never written).
 * b200proj_pose_order_3d fills such an array from the rotations so that slices with nearby
 * planes run together; worthwhile once one batch item's volume no longer fits L2 (about
 * 100 MB), where it turns most DRAM reads of the volume into L2 hits, and harmless below.
 * rot is [B_rot, P, 3, 3] with B_rot 1 or B, exactly as given to the operator. */
int b200proj_pose_order_3d(const float* rot, int64_t B, int64_t B_rot, int64_t P,
                           int32_t* order, void* stream);
int b200proj_pose_order_3d_f64(const double* rot, int64_t B, int64_t B_rot, int64_t P,
                               int32_t* order, void* stream);

/* ---- backward of forward projection ----------------------------------------------------
 * grad_rec [B,(R,)R,Rh] is zero-filled here and accumulated with atomics.
 * grad_rot [B_rot,P,dim,dim] / grad_shifts [B_shift,P,2]: pass NULL when the gradient is
 * not needed (the reference decides this from requires_grad inside the op:
 * csrc/cuda/3d/projection_3d_to_2d_kernels.cu:1066-1067); when given they are zero-filled
 * here.  grad_shifts requires shifts.
 * replaces: project_2d_back_cuda       csrc/cuda/2d/projection_2d_kernels.cu:760-919
 *           project_3d_to_2d_back_cuda csrc/cuda/3d/projection_3d_to_2d_kernels.cu:1018-1179 */
int b200proj_project_2d_back(const float* grad_proj, const float* rec, int64_t B, int64_t R,
                             const float* rot, int64_t B_rot,
                             const float* shifts, int64_t B_shift,
                             int64_t P, int64_t N, int interpolation, double oversampling,
                             double fourier_radius_cutoff,
                             float* grad_rec, float* grad_rot, float* grad_shifts, void* stream);
int b200proj_project_3d_to_2d_back(const float* grad_proj, const float* rec, int64_t B, int64_t R,
                                   const float* rot, int64_t B_rot,
                                   const float* shifts, int64_t B_shift,
                                   int64_t P, int64_t N, int interpolation, double oversampling,
                                   double fourier_radius_cutoff,
                                   float* grad_rec, float* grad_rot, float* grad_shifts,
                                   const int32_t* pose_order, void* stream);

/* ---- back-projection (scatter) ---------------------------------------------------------
 * data_rec [B,(R,)R,Rh] complex and, when weights != NULL, weight_rec (same shape, float)
 * receive the projections / weights; R must equal b200proj_rec_boxsize(N, oversampling).
 * accumulate == 0: both volumes are zero-filled first (the reference's behaviour);
 * accumulate != 0: the call adds into the existing contents (for streaming many chunks of
 * projections into one volume without a per-chunk sum).
 * workspace: optional scratch in device memory, 16-byte aligned, of at least
 * b200proj_backproject_workspace_bytes(...) bytes, or NULL.  With weights and a workspace the
 * kernel accumulates data and weight of each voxel in one 16-byte slot of the workspace (one
 * vector reduction per tap instead of two), then folds the workspace into data_rec /
 * weight_rec; results are the same up to summation order.  Without a workspace (or without
 * weights) it reduces straight into the outputs.  The workspace holds no state between calls.
 * replaces: backproject_2d_forw_cuda       csrc/cuda/2d/backprojection_2d_kernels.cu:827-976
 *           backproject_2d_to_3d_forw_cuda csrc/cuda/3d/backprojection_2d_to_3d_kernels.cu:1001-1188 */
int b200proj_backproject_2d_forw(const float* proj, const float* weights, int64_t B, int64_t R,
                                 const float* rot, int64_t B_rot,
                                 const float* shifts, int64_t B_shift,
                                 int64_t P, int64_t N, int interpolation, double oversampling,
                                 double fourier_radius_cutoff,
                                 float* data_rec, float* weight_rec, int accumulate,
                                 void* workspace, size_t workspace_bytes, void* stream);
int b200proj_backproject_2d_to_3d_forw(const float* proj, const float* weights, int64_t B,
                                       int64_t R, const float* rot, int64_t B_rot,
                                       const float* shifts, int64_t B_shift,
                                       int64_t P, int64_t N, int interpolation,
                                       double oversampling, double fourier_radius_cutoff,
                                       float* data_rec, float* weight_rec, int accumulate,
                                       void* workspace, size_t workspace_bytes, void* stream);

/* Bytes of workspace with which a back-projection of these sizes runs faster, or 0 when a
 * workspace would not help (no weights, or too few slices to pay for two extra passes over
 * the volume).  dim = 2 or 3.  No counterpart in the reference (its kernels use no scratch). */
size_t b200proj_backproject_workspace_bytes(int dim, int64_t B, int64_t R, int64_t P, int64_t N,
                                            int interpolation, int has_weights);

/* ---- back-projection without any allocation --------------------------------------------
 * No counterpart in the reference.  Same result as b200proj_backproject_2d_to_3d_forw with
 * weights (data_rec and weight_rec are both required), for callers that are not allowed to
 * allocate device memory: a plugin inside a host application that hands out one fixed arena
 * at start-up and forbids cudaMalloc afterwards, a service whose GPU memory was partitioned
 * between tenants in advance, or a latency-bound loop that cannot afford the implicit
 * device-wide synchronisation of cudaMalloc / cudaFree.  Such callers can provide inputs and
 * outputs but no workspace, so the 16-byte-per-voxel accumulation volume lives in a
 * statically sized array inside the library (B200PROJ_NOALLOC_MAX_VOXELS * 16 bytes = 2.06 MiB
 * of device memory, held by every GPU that loads the library until the process exits).
 *  - Limit: B*R*R*(R/2+1) <= B200PROJ_NOALLOC_MAX_VOXELS (box 64 for one batch item, i.e.
 *    32-pixel projections at oversampling 2); larger problems are refused with
 *    B200PROJ_ERR_LIMIT before anything is launched.
 *  - The entry point calls no cudaMalloc, cudaFree or allocating library routine.
 *  - The first call on each device looks up the array's device address
 *    (cudaGetSymbolAddress, with that device current) and caches it.  With CUDA's lazy module
 *    loading that lookup can be what loads the library's device code onto the GPU and reserves
 *    the array, i.e. it may block and take device memory.  Make that first call at start-up
 *    (a call with P = 0 does): before the phase in which allocation is forbidden and before any
 *    stream capture begins.  Later calls only enqueue work.
 *  - The cached address belongs to the device context that was current at the first call.  A
 *    process that destroys it (cudaDeviceReset) must not call this entry point afterwards.
 *  - All calls on a device share the one array, which keeps the previous call's sums; each
 *    call clears the part it uses on its stream first.  Two calls that overlap on the GPU
 *    (different streams, or different host threads) race on the array: serialise them. */
#define B200PROJ_NOALLOC_MAX_VOXELS 135168   /* 64 * 64 * 33 */
int b200proj_backproject_2d_to_3d_forw_noalloc(const float* proj, const float* weights, int64_t B,
                                               int64_t R, const float* rot, int64_t B_rot,
                                               const float* shifts, int64_t B_shift,
                                               int64_t P, int64_t N, int interpolation,
                                               double oversampling, double fourier_radius_cutoff,
                                               float* data_rec, float* weight_rec, int accumulate,
                                               void* stream);

/* ---- streaming back-projection into a persistent accumulator ----------------------------
 * No counterpart in the reference (its callers sum the volumes of separate calls:
 * tests/3d/back/test_performance_back_2d_to_3d.py:357-369).  For reconstructions fed chunk by
 * chunk: the caller owns an accumulator of b200proj_accumulator_bytes(B, R) bytes -- one
 * 16-byte (re, im, weight, 0) slot per voxel of [B,R,R,Rh], 16-byte aligned, zero-filled once
 * by the caller (cudaMemsetAsync) -- and every b200proj_backproject_2d_to_3d_accumulate call
 * ADDS its slices into it with one vector reduction per tap (half the reductions of separate
 * data and weight volumes), choosing the slab-ordered kernel by itself when the accumulator
 * exceeds L2.  Nothing is zero-filled or folded per call.  weights are required.
 * b200proj_accumulator_fold writes (accumulate = 0) or adds (accumulate = 1) the sums into
 * the API's data [B,R,R,Rh] complex / weight [B,R,R,Rh] float volumes; the accumulator is
 * left unchanged. */
size_t b200proj_accumulator_bytes(int64_t B, int64_t R);
int b200proj_backproject_2d_to_3d_accumulate(const float* proj, const float* weights, int64_t B,
                                             int64_t R, const float* rot, int64_t B_rot,
                                             const float* shifts, int64_t B_shift,
                                             int64_t P, int64_t N, int interpolation,
                                             double oversampling, double fourier_radius_cutoff,
                                             void* accumulator, void* stream);
int b200proj_accumulator_fold(const void* accumulator, int64_t B, int64_t R, float* data_rec,
                              float* weight_rec, int accumulate, void* stream);
/* The same for voxels [first_voxel, first_voxel + voxel_count) only (all three pointers are the
 * bases of the whole volumes), so that a caller can fold range by range and hand each finished
 * range to a collective while the next one is folded. */
int b200proj_accumulator_fold_range(const void* accumulator, int64_t first_voxel, int64_t voxel_count,
                                    float* data_rec, float* weight_rec, int accumulate, void* stream);

/* The weighted-average reconstruction data / max(weight, eps) (the usual consumer of the two
 * volumes: README.md:152-160 and paper/main.tex:72 of the reference) straight from the
 * accumulator, for voxels [first_voxel, first_voxel + voxel_count): fold and division in one
 * pass.  normalized is the base of a complex [B,R,R,Rh] volume; eps > 0. */
int b200proj_accumulator_fold_normalized(const void* accumulator, int64_t first_voxel, int64_t voxel_count,
                                         double eps, float* normalized, void* stream);

/* Slab by slab.  An accumulator larger than L2 is filled by slab-ordered passes: the planes of
 * the volume (signed coordinate z = -R/2+1 .. R/2, stored at index z < 0 ? z + R : z) are cut
 * into `slabs` runs of `planes_per_slab` consecutive z, and a pass issues only the reductions
 * that land in its own slab.  b200proj_accumulator_slab_plan reports the cut (slabs = 1: the
 * accumulator is small enough to be scattered in one pass).
 * b200proj_backproject_2d_to_3d_accumulate_slabs does the work of
 * b200proj_backproject_2d_to_3d_accumulate for slabs [slab_first, slab_first + slab_count) only:
 * calling it for every slab once, in any order and grouping, adds exactly what the one-call form
 * adds.  Once a slab's pass has run for the caller's last slices, the voxels
 * b200proj_accumulator_slab_voxels reports for it (at most two ranges per batch item, relative to
 * the batch item's first voxel: planes with negative and with non-negative coordinates) are
 * final, so they can be folded (b200proj_accumulator_fold_range) and handed to a collective on
 * another stream while later slabs are still being scattered.  This is how the reduce of
 * multi-GPU partial volumes is overlapped with the tail of the scatter. */
int b200proj_accumulator_slab_plan(int64_t R, int32_t* slabs, int32_t* planes_per_slab);
int b200proj_backproject_2d_to_3d_accumulate_slabs(const float* proj, const float* weights, int64_t B,
                                                   int64_t R, const float* rot, int64_t B_rot,
                                                   const float* shifts, int64_t B_shift,
                                                   int64_t P, int64_t N, int interpolation,
                                                   double oversampling, double fourier_radius_cutoff,
                                                   void* accumulator, int slab_first, int slab_count,
                                                   void* stream);
int b200proj_accumulator_slab_voxels(int64_t R, int slab_first, int slab_count,
                                     int64_t first_voxel[2], int64_t voxel_count[2]);

/* ---- the steps either side of the operators ----------------------------------------------
 * No raw-operator counterpart in the reference, which does them with torch calls in its README
 * and test utilities (README.md:96-160, tests/test_utils.py:174-293).
 * b200proj_pad_fftshift: `batch` real arrays of box n (dims = 2: [n,n]; 3: [n,n,n]) -> box m
 * (even, >= n), zero-padded by lo = (m-n)/2 in front of every axis and rolled so that the
 * real-space centre lands on index 0 -- the array whose real FFT (norm 'forward') is the
 * reconstruction the projection operators read.  b200proj_ifftshift_crop is its adjoint /
 * inverse: box m -> the centred box n of an inverse-transformed reconstruction.  One pass each
 * (every output element written once). */
int b200proj_pad_fftshift(const float* real, int64_t batch, int dims, int64_t n, int64_t m,
                          float* out, void* stream);
int b200proj_ifftshift_crop(const float* full, int64_t batch, int dims, int64_t m, int64_t n,
                            float* out, void* stream);
int b200proj_pad_fftshift_f64(const double* real, int64_t batch, int dims, int64_t n, int64_t m,
                              double* out, void* stream);
int b200proj_ifftshift_crop_f64(const double* full, int64_t batch, int dims, int64_t m, int64_t n,
                                double* out, void* stream);

/* ---- reduction-rate probe (diagnostic) ------------------------------------------------------
 * No counterpart in the reference.  The scatter kernels are bound by the rate at which the memory
 * system retires red.global.add, not by HBM bandwidth; this probe measures that rate for their
 * access patterns so that a benchmark can state it beside the kernels' own rate.  `blocks` blocks
 * of 256 lanes each issue `iterations` reductions to pseudo-random places of `buffer`
 * (buffer_bytes, 16-byte aligned; size it below L2 for the ceiling, far above for the DRAM rate):
 *   0 one random 16-byte slot per lane (v4)      1 lane pairs on adjacent 16-byte slots (v4)
 *   2 lane pairs sharing a 32-byte sector (v4)   3 four lanes on four adjacent 8-byte voxels (v2)
 *   4 one random 8-byte voxel per lane (v2)      5 lane pairs on adjacent 8-byte voxels (v2)
 * The buffer's contents are added to, not preserved. */
int b200proj_reduction_rate_probe(int pattern, float* buffer, size_t buffer_bytes, int blocks,
                                  int iterations, void* stream);
/* The same probe with the memory traffic of the slab-ordered scatter (pattern 1 otherwise): the lane
 * pairs of block b work inside window  b * n_windows / blocks  of `target` (windows of window_bytes,
 * sized to fit L2; target far beyond L2), so the window moves through the target as the grid
 * advances and every slot is filled from and written back to HBM once, and every lane reads 8 bytes
 * per four reductions from `source` (source_bytes, beyond L2; read cyclically) with streaming
 * loads.  With blocks * 256 * iterations = 16 reductions per 16-byte slot of the target this moves
 * 2 + 2 bytes per reduction through HBM, as that kernel does per tap.  `source` must hold finite numbers (they are
 * added to the target's second and third floats); the target's contents are added to. */
int b200proj_reduction_rate_probe_streaming(float* target, size_t target_bytes, size_t window_bytes,
                                            const float* source, size_t source_bytes, int blocks,
                                            int iterations, int evict_last, void* stream);

/* ---- forward projection that keeps what its backward pass needs ---------------------------
 * No counterpart in the reference (its backward gathers the volume a second time for the pose
 * gradients).  _forw_saving writes the projections [B,P,N,Nh] and, besides, the derivatives of every
 * pixel inside the cutoff with respect to its sample position (c, r[, d]), shift phase applied:
 * derivatives = dim planes of [B,P,N,Nh] complex (dim * B*P*N*Nh*8 bytes, dim = 2 for the 2D pair and 3
 * for the 3D pair; pixels outside the cutoff are left unwritten and are never read).  _back_saved is the backward pass from those: grad_rot from
 * grad_proj and the derivatives, grad_shifts from grad_proj and the saved projections `out`, and --
 * when grad_rec is not NULL -- the same scatter of grad_proj into grad_rec [B,(R,)R,Rh] as
 * b200proj_project_{2d,3d_to_2d}_back (all outputs zero-filled here; NULL = not needed).  Same values as
 * the plain pair of entry points up to rounding (~1e-7); fp32 only. */
int b200proj_project_2d_forw_saving(const float* rec, int64_t B, int64_t R, const float* rot,
                                    int64_t B_rot, const float* shifts, int64_t B_shift, int64_t P,
                                    int64_t N, int interpolation, double oversampling,
                                    double fourier_radius_cutoff, float* out, float* derivatives,
                                    void* stream);
int b200proj_project_2d_back_saved(const float* grad_proj, const float* out, const float* derivatives,
                                   int64_t B, int64_t R, const float* rot, int64_t B_rot,
                                   const float* shifts, int64_t B_shift, int64_t P, int64_t N,
                                   int interpolation, double oversampling, double fourier_radius_cutoff,
                                   float* grad_rec, float* grad_rot, float* grad_shifts, void* stream);
int b200proj_project_3d_to_2d_forw_saving(const float* rec, int64_t B, int64_t R, const float* rot,
                                          int64_t B_rot, const float* shifts, int64_t B_shift, int64_t P,
                                          int64_t N, int interpolation, double oversampling,
                                          double fourier_radius_cutoff, float* out, float* derivatives,
                                          const int32_t* pose_order, void* stream);
int b200proj_project_3d_to_2d_back_saved(const float* grad_proj, const float* out, const float* derivatives,
                                         int64_t B, int64_t R, const float* rot, int64_t B_rot,
                                         const float* shifts, int64_t B_shift, int64_t P, int64_t N,
                                         int interpolation, double oversampling,
                                         double fourier_radius_cutoff, float* grad_rec, float* grad_rot,
                                         float* grad_shifts, const int32_t* pose_order, void* stream);

/* ---- backward of back-projection (gather) ----------------------------------------------
 * grad_proj [B,P,N,Nh] complex is fully written.  grad_weights [B,P,N,Nh] float is written
 * only when grad_weight_rec and grad_weights are both non-NULL (always tri/bi-linear).
 * grad_rot / grad_shifts as above (NULL = not needed; zero-filled here when given).
 * replaces: backproject_2d_back_cuda       csrc/cuda/2d/backprojection_2d_kernels.cu:979-1190
 *           backproject_2d_to_3d_back_cuda csrc/cuda/3d/backprojection_2d_to_3d_kernels.cu:1191-1404 */
int b200proj_backproject_2d_back(const float* grad_data_rec, const float* grad_weight_rec,
                                 const float* proj, int64_t B, int64_t R,
                                 const float* rot, int64_t B_rot,
                                 const float* shifts, int64_t B_shift,
                                 int64_t P, int64_t N, int interpolation, double oversampling,
                                 double fourier_radius_cutoff,
                                 float* grad_proj, float* grad_weights, float* grad_rot,
                                 float* grad_shifts, void* stream);
int b200proj_backproject_2d_to_3d_back(const float* grad_data_rec, const float* grad_weight_rec,
                                       const float* proj, int64_t B, int64_t R,
                                       const float* rot, int64_t B_rot,
                                       const float* shifts, int64_t B_shift,
                                       int64_t P, int64_t N, int interpolation,
                                       double oversampling, double fourier_radius_cutoff,
                                       float* grad_proj, float* grad_weights, float* grad_rot,
                                       float* grad_shifts, const int32_t* pose_order, void* stream);


/* ---- complex128 / float64 variants ------------------------------------------------------
 * The same eight operators for double precision tensors (complex128 data, float64 poses and
 * weights): identical arguments with `double` in place of `float`.  The reference's CUDA
 * wrappers serve these dtypes by copying to the host and running its CPU kernels
 * (csrc/cuda/3d/projection_3d_to_2d_kernels.cu:902-918, used by its gradcheck tests); here they
 * run on the GPU with the same kernels instantiated for double.  Reductions use
 * red.global.add.f64; the workspace arguments of the back-projection entries are accepted and
 * ignored (the interleaved and slab-ordered paths are fp32 only). */
int b200proj_project_2d_forw_f64(const double* rec, int64_t B, int64_t R,
                             const double* rot, int64_t B_rot,
                             const double* shifts, int64_t B_shift,
                             int64_t P, int64_t N, int interpolation, double oversampling,
                             double fourier_radius_cutoff, double* out, void* stream);
int b200proj_project_3d_to_2d_forw_f64(const double* rec, int64_t B, int64_t R,
                                   const double* rot, int64_t B_rot,
                                   const double* shifts, int64_t B_shift,
                                   int64_t P, int64_t N, int interpolation, double oversampling,
                                   double fourier_radius_cutoff, double* out,
                                   const int32_t* pose_order, void* stream);
int b200proj_project_2d_back_f64(const double* grad_proj, const double* rec, int64_t B, int64_t R,
                             const double* rot, int64_t B_rot,
                             const double* shifts, int64_t B_shift,
                             int64_t P, int64_t N, int interpolation, double oversampling,
                             double fourier_radius_cutoff,
                             double* grad_rec, double* grad_rot, double* grad_shifts, void* stream);
int b200proj_project_3d_to_2d_back_f64(const double* grad_proj, const double* rec, int64_t B, int64_t R,
                                   const double* rot, int64_t B_rot,
                                   const double* shifts, int64_t B_shift,
                                   int64_t P, int64_t N, int interpolation, double oversampling,
                                   double fourier_radius_cutoff,
                                   double* grad_rec, double* grad_rot, double* grad_shifts,
                                   const int32_t* pose_order, void* stream);
int b200proj_backproject_2d_forw_f64(const double* proj, const double* weights, int64_t B, int64_t R,
                                 const double* rot, int64_t B_rot,
                                 const double* shifts, int64_t B_shift,
                                 int64_t P, int64_t N, int interpolation, double oversampling,
                                 double fourier_radius_cutoff,
                                 double* data_rec, double* weight_rec, int accumulate,
                                 void* workspace, size_t workspace_bytes, void* stream);
int b200proj_backproject_2d_to_3d_forw_f64(const double* proj, const double* weights, int64_t B,
                                       int64_t R, const double* rot, int64_t B_rot,
                                       const double* shifts, int64_t B_shift,
                                       int64_t P, int64_t N, int interpolation,
                                       double oversampling, double fourier_radius_cutoff,
                                       double* data_rec, double* weight_rec, int accumulate,
                                       void* workspace, size_t workspace_bytes, void* stream);
int b200proj_backproject_2d_back_f64(const double* grad_data_rec, const double* grad_weight_rec,
                                 const double* proj, int64_t B, int64_t R,
                                 const double* rot, int64_t B_rot,
                                 const double* shifts, int64_t B_shift,
                                 int64_t P, int64_t N, int interpolation, double oversampling,
                                 double fourier_radius_cutoff,
                                 double* grad_proj, double* grad_weights, double* grad_rot,
                                 double* grad_shifts, void* stream);
int b200proj_backproject_2d_to_3d_back_f64(const double* grad_data_rec, const double* grad_weight_rec,
                                       const double* proj, int64_t B, int64_t R,
                                       const double* rot, int64_t B_rot,
                                       const double* shifts, int64_t B_shift,
                                       int64_t P, int64_t N, int interpolation,
                                       double oversampling, double fourier_radius_cutoff,
                                       double* grad_proj, double* grad_weights, double* grad_rot,
                                       double* grad_shifts, const int32_t* pose_order, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200PROJ_H */
