// C ABI of the sm_100a Fourier-slice operators: argument validation, geometry set-up,
// zero-fill of atomically accumulated outputs and kernel dispatch.  Declarations and the
// reference interfaces each entry point replaces are in include/b200proj.h.
#include "b200proj.h"

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <climits>
#include <cstdint>
#include <mutex>
#include <type_traits>

#include "fourier_slice_kernels.cuh"

namespace {

using namespace b200proj;

thread_local char g_error[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

int cuda_fail(cudaError_t e, const char* what) {
    return fail(B200PROJ_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

struct Launch {
    SliceGeom g;
    dim3 grid;
    int64_t B, P;
    size_t rec_count;    // voxels in [B, (R,) R, Rh]
    size_t pix_count;    // pixels in [B, P, N, Nh]
};

// Validate the arguments common to all operators and derive the kernel geometry.
int prepare(Launch& L, int dim, int64_t B, int64_t R, int64_t B_rot, const void* rot,
            const void* shifts, int64_t B_shift, int64_t P, int64_t N, int interpolation,
            double oversampling, double cutoff) {
    g_error[0] = 0;
    if (interpolation != B200PROJ_LINEAR && interpolation != B200PROJ_CUBIC)
        return fail(B200PROJ_ERR_ARGUMENT, "Supported interpolation methods: 'linear', 'cubic'");
    if (B < 1 || P < 0) return fail(B200PROJ_ERR_ARGUMENT, "batch size must be >= 1 and pose count >= 0 (B=%lld, P=%lld)", (long long)B, (long long)P);
    if (N < 2 || (N % 2) != 0) return fail(B200PROJ_ERR_ARGUMENT, "projection boxsize (%lld) must be even and >= 2", (long long)N);
    if (R < 2 || (R % 2) != 0) return fail(B200PROJ_ERR_ARGUMENT, "reconstruction boxsize (%lld) must be even and >= 2", (long long)R);
    if (rot == nullptr) return fail(B200PROJ_ERR_ARGUMENT, "rotations pointer is NULL");
    if (B_rot != 1 && B_rot != B) return fail(B200PROJ_ERR_ARGUMENT, "Batch size of rotations must be 1 or same as reconstruction (B_rot=%lld, B=%lld)", (long long)B_rot, (long long)B);
    if (shifts != nullptr && B_shift != 1 && B_shift != B)
        return fail(B200PROJ_ERR_ARGUMENT, "Batch size of shifts must be 1 or same as reconstruction (B_shift=%lld, B=%lld)", (long long)B_shift, (long long)B);
    if (!(oversampling > 0.0) || !std::isfinite(oversampling))
        return fail(B200PROJ_ERR_ARGUMENT, "oversampling must be a positive finite number");
    if (std::isnan(cutoff)) return fail(B200PROJ_ERR_ARGUMENT, "fourier_radius_cutoff is NaN");
    if ((double)N * oversampling > 1073741824.0)
        return fail(B200PROJ_ERR_LIMIT, "N * oversampling = %g puts sample coordinates beyond 2^30", (double)N * oversampling);

    const int64_t Nh = N / 2 + 1, Rh = R / 2 + 1;
    const int64_t vol = (dim == 3 ? R : 1) * R * Rh;
    if (vol > INT_MAX) return fail(B200PROJ_ERR_LIMIT, "reconstruction of box %lld exceeds 2^31-1 voxels per batch item", (long long)R);
    if (N > 2048) return fail(B200PROJ_ERR_LIMIT, "projection boxsize %lld exceeds 2048", (long long)N);
    if (P * dim * dim > INT_MAX / 2) return fail(B200PROJ_ERR_LIMIT, "too many poses per batch item (%lld)", (long long)P);

    SliceGeom& g = L.g;
    g.N = (int)N; g.Nh = (int)Nh; g.R = (int)R; g.Rh = (int)Rh; g.half = (int)(R / 2);
    g.P = (int)P;
    g.tiles_j = (int)((Nh + kTileJ - 1) / kTileJ);
    g.tiles_i = (int)((N + kTileI - 1) / kTileI);
    g.rot_stride_b = (B_rot == 1) ? 0 : (int)(P * dim * dim);
    g.has_shift = shifts != nullptr;
    g.shift_stride_b = (!g.has_shift || B_shift == 1) ? 0 : (int)(P * 2);
    const float rc = (float)cutoff;
    g.cutoff_sq = rc * rc;
    g.cutoff_sq_d = cutoff * cutoff;
    g.os = oversampling;
    g.phase_scale = -2.0 * M_PI / (double)(float)N;
    g.shift_scale = -2.0 * M_PI / (double)N;
    g.vol_elems = vol;
    g.order = nullptr;
    g.pack_index = nullptr;
    g.pack_count = 0;
    g.replicas = 1;
    g.replica_stride = 0;

    if (B * P > INT_MAX / 2) return fail(B200PROJ_ERR_LIMIT, "B*P = %lld slices exceed the grid limit; split the poses into chunks", (long long)(B * P));
    g.BP = (int)(B * P);
    g.slice_pixels = (int)(N * Nh);
    g.os_f = (float)oversampling;
    g.os_is_float = ((double)g.os_f == oversampling);
    g.sparse_samples = oversampling >= 1.5;
    // exact for tile < 2^16 whenever tiles_j <= 2^16 (the numbers of tiles per slice are far below)
    g.tiles_j_magic = g.tiles_j == 1 ? 0u : (unsigned)(((1ull << 32) + (unsigned long long)g.tiles_j - 1) / (unsigned long long)g.tiles_j);
    // x = tile, (y, z) = the slice (see block_work for the three decodings)
    unsigned gy, gz;
    if (B > 1 && P >= 1 && P <= 32768 && B <= 65535) {
        g.decode = 1;
        gy = (unsigned)P;
        gz = (unsigned)B;
    } else {
        g.decode = (B == 1) ? 0 : 2;
        const int64_t bp = B * P;
        gy = (unsigned)(bp < 32768 ? (bp > 0 ? bp : 1) : 32768);
        gz = (unsigned)((bp + 32767) / 32768 > 0 ? (bp + 32767) / 32768 : 1);
    }
    L.grid = dim3((unsigned)(g.tiles_j * g.tiles_i), gy, gz);
    L.B = B; L.P = P;
    L.rec_count = (size_t)B * (size_t)vol;
    L.pix_count = (size_t)B * (size_t)P * (size_t)N * (size_t)Nh;
    return B200PROJ_OK;
}

int check_launch(const char* what) {
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? B200PROJ_OK : cuda_fail(e, what);
}

int zero_async(void* p, size_t bytes, cudaStream_t s) {
    if (p == nullptr || bytes == 0) return B200PROJ_OK;
    const cudaError_t e = cudaMemsetAsync(p, 0, bytes, s);
    return e == cudaSuccess ? B200PROJ_OK : cuda_fail(e, "cudaMemsetAsync");
}

// Slab plan of the slab-ordered 3D back-projection: volumes whose planes of one batch item
// exceed 160 MB are processed in slabs of at most `slab_mb` MB of planes.  `eager` lowers the
// threshold to 120 MB: an interleaved accumulator (16 bytes per voxel) just above L2 (box 256:
// 135 MB) loses its sectors between hits when the samples are sparse (linear taps at oversampling
// >= 1.5: 4.4x the compulsory DRAM traffic in one pass), and two slab passes then cost less than
// that (11.2 -> 10.65 ms per 50,000 slices); with dense samples (oversampling 1) or cubic footprints
// the second visit of the pixels costs more than the evictions (measured 6 % and 1.5 % slower).
// Tunable for experiments through B200PROJ_SLAB_MB / B200PROJ_SLAB_MIN_MB /
// B200PROJ_SLAB_MIN_MB_EAGER (read once).
struct SlabPlan { int slabs, planes; };
SlabPlan slab_plan(int64_t R, bool has_weights, bool interleaved = false, bool eager = false) {
    static const double slab_mb = [] { const char* e = getenv("B200PROJ_SLAB_MB"); return e ? atof(e) : 64.0; }();
    static const double min_mb = [] { const char* e = getenv("B200PROJ_SLAB_MIN_MB"); return e ? atof(e) : 160.0; }();
    static const double min_mb_e = [] { const char* e = getenv("B200PROJ_SLAB_MIN_MB_EAGER"); return e ? atof(e) : 120.0; }();
    const double plane_bytes = (double)R * (double)(R / 2 + 1) * (interleaved ? 16.0 : has_weights ? 12.0 : 8.0);
    const double threshold = (eager && min_mb_e < min_mb) ? min_mb_e : min_mb;
    if (slab_mb <= 0.0 || plane_bytes * (double)R <= threshold * 1e6) return {1, (int)R};
    // 16-byte voxels: fewer, larger reductions per plane leave room for 1.4x the bytes (measured)
    int planes = (int)(slab_mb * (interleaved ? 1.4 : 1.0) * 1e6 / plane_bytes);
    if (planes < 1) planes = 1;
    const int slabs = (int)((R + planes - 1) / planes);
    return {slabs, planes};
}

// Copies of a small interleaved workspace over which the slices of one call are spread: reductions
// onto less than ~2 MB run at 55-60 % of the rate they reach on a larger target (probe: 146 instead
// of 254 G taps/s at 128 KB), so a reconstruction of `bytes` bytes gets the power of two of copies
// that brings it to 2 MiB, at most 32 and at most one per 32 slices.
int workspace_replicas(double bytes, int64_t P) {
    int r = 1;
    while (r < 32 && bytes * r < 2097152.0 && P >= 32 * (int64_t)(2 * r)) r *= 2;
    return r;
}

// Launch the slab-ordered kernel into an interleaved accumulator for slabs [first, first + count).
void launch_slab_interleaved(const Launch& L, cudaStream_t s, bool cubic, const float* proj, const float* weights,
                             const float* rot, const float* shifts, float4* acc, const SlabPlan& plan, int first, int count) {
    const dim3 grid((unsigned)(L.B * L.P), (unsigned)count, 1);
    if (cubic)
        backproject_slab_kernel<true, true, true><<<grid, kBlockThreads, 0, s>>>((const float2*)proj, weights, rot, shifts, nullptr, nullptr, acc, L.g, plan.planes, first);
    else
        backproject_slab_kernel<false, true, true><<<grid, kBlockThreads, 0, s>>>((const float2*)proj, weights, rot, shifts, nullptr, nullptr, acc, L.g, plan.planes, first);
}

// Linear forward projection with two pixels per lane (project_forw_rows2_kernel); B200PROJ_LINEAR_ROWS2=0
// selects the one-pixel kernel for comparisons (read once).
bool linear_rows2() {
    static const bool on = [] { const char* e = getenv("B200PROJ_LINEAR_ROWS2"); return e ? atoi(e) != 0 : true; }();
    return on;
}

// ---- operator bodies, templated on the dimensionality and the real type (float | double) ------------------------------------
template <int DIM, typename Real>
int project_forw(const Real* rec, int64_t B, int64_t R, const Real* rot, int64_t B_rot,
                 const Real* shifts, int64_t B_shift, int64_t P, int64_t N, int interpolation,
                 double os, double cutoff, Real* out, const int32_t* pose_order, void* stream) {
    Launch L;
    if (int rc = prepare(L, DIM, B, R, B_rot, rot, shifts, B_shift, P, N, interpolation, os, cutoff)) return rc;
    if (rec == nullptr || out == nullptr) return fail(B200PROJ_ERR_ARGUMENT, "reconstruction / output pointer is NULL");
    L.g.order = pose_order;
    if (P == 0) return B200PROJ_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const C2<Real>* v = (const C2<Real>*)rec;
    C2<Real>* o = (C2<Real>*)out;
    if (interpolation == B200PROJ_CUBIC) {
        project_forw_kernel<DIM, true><<<L.grid, kBlockThreads, 0, s>>>(v, rot, shifts, o, L.g);
    } else if (linear_rows2()) {
        // linear: two pixels per lane, a block covers 16 columns x 32 rows
        const dim3 grid((unsigned)(L.g.tiles_j * ((N + 2 * kTileI - 1) / (2 * kTileI))), L.grid.y, L.grid.z);
        project_forw_rows2_kernel<DIM><<<grid, kBlockThreads, 0, s>>>(v, rot, shifts, o, L.g);
    } else {
        project_forw_kernel<DIM, false><<<L.grid, kBlockThreads, 0, s>>>(v, rot, shifts, o, L.g);
    }
    return check_launch("project_forw launch");
}

template <int DIM, bool CUBIC, typename Real>
void launch_project_back(const Launch& L, cudaStream_t s, const C2<Real>* gp, const C2<Real>* rec,
                         const Real* rot, const Real* shifts, C2<Real>* grad_rec, Real* grad_rot,
                         Real* grad_shift) {
    const bool nr = grad_rot != nullptr, ns = grad_shift != nullptr;
#define B200PROJ_PB(NR, NS) \
    project_back_kernel<DIM, CUBIC, NR, NS><<<L.grid, kBlockThreads, 0, s>>>(gp, rec, rot, shifts, grad_rec, grad_rot, grad_shift, L.g)
    if (nr && ns) B200PROJ_PB(true, true);
    else if (nr) B200PROJ_PB(true, false);
    else if (ns) B200PROJ_PB(false, true);
    else B200PROJ_PB(false, false);
#undef B200PROJ_PB
}

template <int DIM, bool CUBIC, bool NEED_REC>
void launch_project_back_saved(const Launch& L, cudaStream_t s, const float2* gp, const float2* out, const float2* derivs,
                               const float* rot, const float* shifts, float2* grad_rec, float* grad_rot, float* grad_shift) {
    const bool nr = grad_rot != nullptr, ns = grad_shift != nullptr;
#define B200PROJ_PBS(NR, NS) \
    project_back_saved_kernel<DIM, CUBIC, NR, NS, NEED_REC><<<L.grid, kBlockThreads, 0, s>>>(gp, out, derivs, rot, shifts, grad_rec, grad_rot, grad_shift, L.g)
    if (nr && ns) B200PROJ_PBS(true, true);
    else if (nr) B200PROJ_PBS(true, false);
    else if (ns) B200PROJ_PBS(false, true);
    else B200PROJ_PBS(false, false);
#undef B200PROJ_PBS
}

// Forward projection that also writes the pixels' derivatives, and the backward pass from them (fp32).
template <int DIM>
int project_forw_saving(const float* rec, int64_t B, int64_t R, const float* rot, int64_t B_rot, const float* shifts,
                        int64_t B_shift, int64_t P, int64_t N, int interpolation, double os, double cutoff,
                        float* out, float* derivatives, const int32_t* pose_order, void* stream) {
    Launch L;
    if (int rc = prepare(L, DIM, B, R, B_rot, rot, shifts, B_shift, P, N, interpolation, os, cutoff)) return rc;
    if (rec == nullptr || out == nullptr || derivatives == nullptr) return fail(B200PROJ_ERR_ARGUMENT, "reconstruction / output / derivatives pointer is NULL");
    L.g.order = pose_order;
    if (P == 0) return B200PROJ_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (interpolation == B200PROJ_CUBIC)
        project_forw_saving_kernel<DIM, true><<<L.grid, kBlockThreads, 0, s>>>((const float2*)rec, rot, shifts, (float2*)out, (float2*)derivatives, L.g);
    else
        project_forw_saving_kernel<DIM, false><<<L.grid, kBlockThreads, 0, s>>>((const float2*)rec, rot, shifts, (float2*)out, (float2*)derivatives, L.g);
    return check_launch("project_forw (saving derivatives) launch");
}

template <int DIM>
int project_back_saved(const float* grad_proj, const float* out, const float* derivatives, int64_t B, int64_t R,
                       const float* rot, int64_t B_rot, const float* shifts, int64_t B_shift, int64_t P, int64_t N,
                       int interpolation, double os, double cutoff, float* grad_rec, float* grad_rot, float* grad_shifts,
                       const int32_t* pose_order, void* stream) {
    Launch L;
    if (int rc = prepare(L, DIM, B, R, B_rot, rot, shifts, B_shift, P, N, interpolation, os, cutoff)) return rc;
    L.g.order = pose_order;
    if (grad_proj == nullptr) return fail(B200PROJ_ERR_ARGUMENT, "grad_projections pointer is NULL");
    if (grad_rot != nullptr && derivatives == nullptr) return fail(B200PROJ_ERR_ARGUMENT, "grad_rotations requested but no saved derivatives given");
    if (grad_shifts != nullptr && (shifts == nullptr || out == nullptr))
        return fail(B200PROJ_ERR_ARGUMENT, "grad_shifts requested but no shifts / saved projections given");
    if (grad_rec == nullptr && grad_rot == nullptr && grad_shifts == nullptr) return B200PROJ_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (int rc = zero_async(grad_rec, L.rec_count * sizeof(float2), s)) return rc;
    if (int rc = zero_async(grad_rot, (size_t)B_rot * P * DIM * DIM * sizeof(float), s)) return rc;
    if (int rc = zero_async(grad_shifts, (size_t)(shifts ? B_shift : 0) * P * 2 * sizeof(float), s)) return rc;
    if (P == 0) return B200PROJ_OK;
    const float2* gp = (const float2*)grad_proj;
    const float2* o = (const float2*)out;
    const float2* d = (const float2*)derivatives;
    const bool cubic = interpolation == B200PROJ_CUBIC;
    if (grad_rec != nullptr) {
        if (cubic) launch_project_back_saved<DIM, true, true>(L, s, gp, o, d, rot, shifts, (float2*)grad_rec, grad_rot, grad_shifts);
        else launch_project_back_saved<DIM, false, true>(L, s, gp, o, d, rot, shifts, (float2*)grad_rec, grad_rot, grad_shifts);
    } else {
        launch_project_back_saved<DIM, false, false>(L, s, gp, o, d, rot, shifts, nullptr, grad_rot, grad_shifts);
    }
    return check_launch("project_back (saved derivatives) launch");
}

template <int DIM, typename Real>
int project_back(const Real* grad_proj, const Real* rec, int64_t B, int64_t R, const Real* rot,
                 int64_t B_rot, const Real* shifts, int64_t B_shift, int64_t P, int64_t N,
                 int interpolation, double os, double cutoff, Real* grad_rec, Real* grad_rot,
                 Real* grad_shifts, const int32_t* pose_order, void* stream) {
    Launch L;
    if (int rc = prepare(L, DIM, B, R, B_rot, rot, shifts, B_shift, P, N, interpolation, os, cutoff)) return rc;
    L.g.order = pose_order;
    if (grad_proj == nullptr || rec == nullptr || grad_rec == nullptr)
        return fail(B200PROJ_ERR_ARGUMENT, "grad_projections / reconstruction / grad_reconstruction pointer is NULL");
    if (grad_shifts != nullptr && shifts == nullptr)
        return fail(B200PROJ_ERR_ARGUMENT, "grad_shifts requested but no shifts given");
    cudaStream_t s = (cudaStream_t)stream;
    if (int rc = zero_async(grad_rec, L.rec_count * sizeof(C2<Real>), s)) return rc;
    if (int rc = zero_async(grad_rot, (size_t)B_rot * P * DIM * DIM * sizeof(Real), s)) return rc;
    if (int rc = zero_async(grad_shifts, (size_t)(shifts ? B_shift : 0) * P * 2 * sizeof(Real), s)) return rc;
    if (P == 0) return B200PROJ_OK;
    if (interpolation == B200PROJ_CUBIC)
        launch_project_back<DIM, true>(L, s, (const C2<Real>*)grad_proj, (const C2<Real>*)rec, rot, shifts, (C2<Real>*)grad_rec, grad_rot, grad_shifts);
    else
        launch_project_back<DIM, false>(L, s, (const C2<Real>*)grad_proj, (const C2<Real>*)rec, rot, shifts, (C2<Real>*)grad_rec, grad_rot, grad_shifts);
    return check_launch("project_back launch");
}

template <int DIM, typename Real>
int backproject_forw(const Real* proj, const Real* weights, int64_t B, int64_t R,
                     const Real* rot, int64_t B_rot, const Real* shifts, int64_t B_shift,
                     int64_t P, int64_t N, int interpolation, double os, double cutoff,
                     Real* data_rec, Real* weight_rec, int accumulate, void* workspace,
                     size_t workspace_bytes, void* stream) {
    Launch L;
    if (int rc = prepare(L, DIM, B, R, B_rot, rot, shifts, B_shift, P, N, interpolation, os, cutoff)) return rc;
    if (proj == nullptr || data_rec == nullptr) return fail(B200PROJ_ERR_ARGUMENT, "projections / data_reconstruction pointer is NULL");
    if ((weights != nullptr) != (weight_rec != nullptr))
        return fail(B200PROJ_ERR_ARGUMENT, "weights and weight_reconstruction must be given together");
    if (R != b200proj_rec_boxsize(N, os))
        return fail(B200PROJ_ERR_ARGUMENT, "reconstruction boxsize %lld does not match ceil(N*oversampling) rounded up to even = %lld",
                    (long long)R, (long long)b200proj_rec_boxsize(N, os));
    cudaStream_t s = (cudaStream_t)stream;
    const bool cubic = interpolation == B200PROJ_CUBIC, hw = weights != nullptr;
    // Interleaved path: data and weight of a voxel share one 16-byte slot of the workspace
    // (one v4 reduction per tap), folded into the outputs afterwards.
    const size_t ws_one = L.rec_count * sizeof(float4);
    constexpr bool kIsF32 = std::is_same<Real, float>::value;  // workspace and slab paths exist in fp32 only
    if constexpr (kIsF32) {
    if (hw && P > 0 && !(DIM == 3 && slab_plan(R, hw).slabs > 1) && workspace != nullptr && workspace_bytes >= ws_one &&
        (reinterpret_cast<uintptr_t>(workspace) & 15u) == 0) {
        // small reconstructions: as many copies as the rule wants and the workspace holds
        int replicas = workspace_replicas((double)ws_one, P);
        while (replicas > 1 && (size_t)replicas * ws_one > workspace_bytes) replicas /= 2;
        L.g.replicas = replicas;
        L.g.replica_stride = (long long)L.rec_count;
        const size_t ws_need = (size_t)replicas * ws_one;
        if (int rc = zero_async(workspace, ws_need, s)) return rc;
        float4* acc = (float4*)workspace;
        const SlabPlan plan_i = (DIM == 3) ? slab_plan(R, true, true, /*eager=*/!cubic && os >= 1.5) : SlabPlan{1, (int)R};
        if (DIM == 3 && plan_i.slabs > 1)      // the 16-byte volume itself is beyond L2: slab-ordered passes
            launch_slab_interleaved(L, s, cubic, (const float*)proj, (const float*)weights, (const float*)rot, (const float*)shifts, acc, plan_i, 0, plan_i.slabs);
        else if (cubic)
            backproject_forw_interleaved_kernel<DIM, true><<<L.grid, kBlockThreads, 0, s>>>((const C2<Real>*)proj, weights, rot, shifts, acc, L.g);
        else
            backproject_forw_interleaved_kernel<DIM, false><<<L.grid, kBlockThreads, 0, s>>>((const C2<Real>*)proj, weights, rot, shifts, acc, L.g);
        if (int rc = check_launch("backproject_forw (interleaved) launch")) return rc;
        const size_t blocks = (L.rec_count + 255) / 256;
        fold_interleaved_kernel<<<(unsigned)(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0, s>>>(acc, (C2<Real>*)data_rec, weight_rec, L.rec_count, accumulate != 0,
                                                                                              replicas, L.rec_count);
        return check_launch("fold_interleaved launch");
    }
    }
    if (!accumulate) {
        if (int rc = zero_async(data_rec, L.rec_count * sizeof(C2<Real>), s)) return rc;
        if (int rc = zero_async(weight_rec, L.rec_count * sizeof(Real), s)) return rc;
    }
    if (P == 0) return B200PROJ_OK;
    const C2<Real>* p = (const C2<Real>*)proj;
    C2<Real>* d = (C2<Real>*)data_rec;
    if constexpr (DIM == 3 && kIsF32) {
        // volumes beyond L2: slab-ordered passes that keep the active planes L2-resident
        const SlabPlan plan = slab_plan(R, hw);
        if (plan.slabs > 1) {
            const dim3 grid((unsigned)(B * P), (unsigned)plan.slabs, 1);
#define B200PROJ_SL(C, W) \
    backproject_slab_kernel<C, W><<<grid, kBlockThreads, 0, s>>>(p, weights, rot, shifts, d, weight_rec, nullptr, L.g, plan.planes, 0)
            if (cubic && hw) B200PROJ_SL(true, true);
            else if (cubic) B200PROJ_SL(true, false);
            else if (hw) B200PROJ_SL(false, true);
            else B200PROJ_SL(false, false);
#undef B200PROJ_SL
            return check_launch("backproject_forw (slab-ordered) launch");
        }
    }
#define B200PROJ_BP(C, W) \
    backproject_forw_kernel<DIM, C, W><<<L.grid, kBlockThreads, 0, s>>>(p, weights, rot, shifts, d, weight_rec, L.g)
    if (cubic && hw) B200PROJ_BP(true, true);
    else if (cubic) B200PROJ_BP(true, false);
    else if (hw) B200PROJ_BP(false, true);
    else B200PROJ_BP(false, false);
#undef B200PROJ_BP
    return check_launch("backproject_forw launch");
}

template <int DIM, bool CUBIC, typename Real>
void launch_backproject_back(const Launch& L, cudaStream_t s, const C2<Real>* gd, const Real* gw,
                             const C2<Real>* proj, const Real* rot, const Real* shifts,
                             C2<Real>* grad_proj, Real* grad_weights, Real* grad_rot,
                             Real* grad_shift) {
    const bool nr = grad_rot != nullptr, ns = grad_shift != nullptr;
#define B200PROJ_BB(NR, NS) \
    backproject_back_kernel<DIM, CUBIC, NR, NS><<<L.grid, kBlockThreads, 0, s>>>(gd, gw, proj, rot, shifts, grad_proj, grad_weights, grad_rot, grad_shift, L.g)
    if (nr && ns) B200PROJ_BB(true, true);
    else if (nr) B200PROJ_BB(true, false);
    else if (ns) B200PROJ_BB(false, true);
    else B200PROJ_BB(false, false);
#undef B200PROJ_BB
}

template <int DIM, typename Real>
int backproject_back(const Real* grad_data_rec, const Real* grad_weight_rec, const Real* proj,
                     int64_t B, int64_t R, const Real* rot, int64_t B_rot, const Real* shifts,
                     int64_t B_shift, int64_t P, int64_t N, int interpolation, double os,
                     double cutoff, Real* grad_proj, Real* grad_weights, Real* grad_rot,
                     Real* grad_shifts, const int32_t* pose_order, void* stream) {
    Launch L;
    if (int rc = prepare(L, DIM, B, R, B_rot, rot, shifts, B_shift, P, N, interpolation, os, cutoff)) return rc;
    L.g.order = pose_order;
    if (grad_data_rec == nullptr || grad_proj == nullptr)
        return fail(B200PROJ_ERR_ARGUMENT, "grad_data_rec / grad_projections pointer is NULL");
    if ((grad_rot != nullptr || grad_shifts != nullptr) && proj == nullptr)
        return fail(B200PROJ_ERR_ARGUMENT, "projections are needed for rotation / shift gradients");
    if (grad_shifts != nullptr && shifts == nullptr)
        return fail(B200PROJ_ERR_ARGUMENT, "grad_shifts requested but no shifts given");
    if (R != b200proj_rec_boxsize(N, os))
        return fail(B200PROJ_ERR_ARGUMENT, "grad_data_rec boxsize %lld does not match ceil(N*oversampling) rounded up to even = %lld",
                    (long long)R, (long long)b200proj_rec_boxsize(N, os));
    cudaStream_t s = (cudaStream_t)stream;
    if (int rc = zero_async(grad_rot, (size_t)B_rot * P * DIM * DIM * sizeof(Real), s)) return rc;
    if (int rc = zero_async(grad_shifts, (size_t)(shifts ? B_shift : 0) * P * 2 * sizeof(Real), s)) return rc;
    if (grad_weights != nullptr && grad_weight_rec == nullptr)   // weights given, no incoming gradient: zeros
        if (int rc = zero_async(grad_weights, L.pix_count * sizeof(Real), s)) return rc;
    if (P == 0) return B200PROJ_OK;
    if (interpolation == B200PROJ_CUBIC)
        launch_backproject_back<DIM, true>(L, s, (const C2<Real>*)grad_data_rec, grad_weight_rec, (const C2<Real>*)proj, rot, shifts, (C2<Real>*)grad_proj, grad_weights, grad_rot, grad_shifts);
    else
        launch_backproject_back<DIM, false>(L, s, (const C2<Real>*)grad_data_rec, grad_weight_rec, (const C2<Real>*)proj, rot, shifts, (C2<Real>*)grad_proj, grad_weights, grad_rot, grad_shifts);
    return check_launch("backproject_back launch");
}

// Weighted 3D back-projection that ADDS into a persistent interleaved accumulator (16-byte
// (re, im, w, 0) voxels): one v4 reduction per tap, nothing zero-filled or folded per call.
int backproject_accumulate(const float* proj, const float* weights, int64_t B, int64_t R, const float* rot,
                           int64_t B_rot, const float* shifts, int64_t B_shift, int64_t P, int64_t N,
                           int interpolation, double os, double cutoff, void* accumulator,
                           int slab_first, int slab_count, void* stream) {
    Launch L;
    if (int rc = prepare(L, 3, B, R, B_rot, rot, shifts, B_shift, P, N, interpolation, os, cutoff)) return rc;
    if (proj == nullptr || weights == nullptr || accumulator == nullptr)
        return fail(B200PROJ_ERR_ARGUMENT, "projections, weights and accumulator are all required");
    if ((reinterpret_cast<uintptr_t>(accumulator) & 15u) != 0)
        return fail(B200PROJ_ERR_ARGUMENT, "accumulator must be 16-byte aligned");
    if (R != b200proj_rec_boxsize(N, os))
        return fail(B200PROJ_ERR_ARGUMENT, "reconstruction boxsize %lld does not match ceil(N*oversampling) rounded up to even = %lld",
                    (long long)R, (long long)b200proj_rec_boxsize(N, os));
    const SlabPlan plan = slab_plan(R, true, true);
    if (slab_count < 0) { slab_first = 0; slab_count = plan.slabs; }         // all slabs
    if (slab_first < 0 || slab_count < 1 || slab_first + slab_count > plan.slabs)
        return fail(B200PROJ_ERR_ARGUMENT, "slabs [%d, %d) outside the plan of %d slabs", slab_first, slab_first + slab_count, plan.slabs);
    if (P == 0) return B200PROJ_OK;
    cudaStream_t s = (cudaStream_t)stream;
    float4* acc = (float4*)accumulator;
    const bool cubic = interpolation == B200PROJ_CUBIC;
    if (plan.slabs > 1) {
        launch_slab_interleaved(L, s, cubic, proj, weights, rot, shifts, acc, plan, slab_first, slab_count);
        return check_launch("backproject_accumulate (slab-ordered) launch");
    }
    if (cubic)
        backproject_forw_interleaved_kernel<3, true><<<L.grid, kBlockThreads, 0, s>>>((const float2*)proj, weights, rot, shifts, acc, L.g);
    else
        backproject_forw_interleaved_kernel<3, false><<<L.grid, kBlockThreads, 0, s>>>((const float2*)proj, weights, rot, shifts, acc, L.g);
    return check_launch("backproject_accumulate launch");
}

// pad + fftshift (pad != 0) or ifftshift + crop (pad == 0) of `batch` real arrays with `dims` axes.
template <typename Real>
int pad_shift(const Real* in, int64_t batch, int dims, int64_t n, int64_t m, int pad, Real* out, void* stream) {
    g_error[0] = 0;
    if (in == nullptr || out == nullptr) return fail(B200PROJ_ERR_ARGUMENT, "input / output pointer is NULL");
    if (dims != 2 && dims != 3) return fail(B200PROJ_ERR_ARGUMENT, "dims must be 2 or 3");
    if (batch < 1 || n < 1 || m < n || (m % 2) != 0)
        return fail(B200PROJ_ERR_ARGUMENT, "need batch >= 1, 1 <= n <= m and an even padded box (batch=%lld, n=%lld, m=%lld)", (long long)batch, (long long)n, (long long)m);
    const int64_t out_box = pad ? m : n;
    if (m > 8192 || batch * (dims == 3 ? out_box : 1) > 65535 * 32768ll || out_box > 65535)
        return fail(B200PROJ_ERR_LIMIT, "box %lld / batch %lld beyond what one launch indexes", (long long)m, (long long)batch);
    const int64_t gz = batch * (dims == 3 ? out_box : 1);
    if (gz > 65535) return fail(B200PROJ_ERR_LIMIT, "batch * box = %lld exceeds the grid limit; split the batch", (long long)gz);
    const dim3 grid((unsigned)((out_box + 255) / 256), (unsigned)((out_box + 3) / 4), (unsigned)gz), block(64, 4, 1);
    cudaStream_t s = (cudaStream_t)stream;
    const int lo = (int)((m - n) / 2);
    // 16-byte stores when every output row starts on a 16-byte boundary
    const bool vec = (out_box % 4) == 0 && (reinterpret_cast<uintptr_t>(out) & 15u) == 0;
#define B200PROJ_PS(D, P, V) pad_shift_kernel<D, P, V><<<grid, block, 0, s>>>(in, out, (int)n, (int)m, lo, (int)batch)
    if (dims == 3) {
        if (pad) { if (vec) B200PROJ_PS(3, true, true); else B200PROJ_PS(3, true, false); }
        else     { if (vec) B200PROJ_PS(3, false, true); else B200PROJ_PS(3, false, false); }
    } else {
        if (pad) { if (vec) B200PROJ_PS(2, true, true); else B200PROJ_PS(2, true, false); }
        else     { if (vec) B200PROJ_PS(2, false, true); else B200PROJ_PS(2, false, false); }
    }
#undef B200PROJ_PS
    return check_launch("pad_shift launch");
}

template <typename Real>
int pose_order_3d(const Real* rot, int64_t B, int64_t B_rot, int64_t P, int32_t* order, void* stream) {
    g_error[0] = 0;
    if (rot == nullptr || order == nullptr) return fail(B200PROJ_ERR_ARGUMENT, "rotations / order pointer is NULL");
    if (B < 1 || P < 0) return fail(B200PROJ_ERR_ARGUMENT, "batch size must be >= 1 and pose count >= 0 (B=%lld, P=%lld)", (long long)B, (long long)P);
    if (B_rot != 1 && B_rot != B) return fail(B200PROJ_ERR_ARGUMENT, "Batch size of rotations must be 1 or same as reconstruction (B_rot=%lld, B=%lld)", (long long)B_rot, (long long)B);
    if (B * P > INT_MAX / 2 || B > 65535 * 32768ll) return fail(B200PROJ_ERR_LIMIT, "B*P = %lld slices exceed the grid limit; split the poses into chunks", (long long)(B * P));
    if (P == 0) return B200PROJ_OK;
    pose_order_kernel<<<(unsigned)B, kOrderBins, 0, (cudaStream_t)stream>>>(rot, B_rot == 1 ? 0ll : (long long)P * 9, (int)P, order);
    return check_launch("pose_order launch");
}

// ---- built-in scratch of the allocation-free back-projection entry point -----------------
// The array lives in every GPU context that loads this library, from load until exit.
constexpr long long kNoAllocMaxVoxels = B200PROJ_NOALLOC_MAX_VOXELS;
static __device__ __align__(256) float4 g_noalloc_accum[kNoAllocMaxVoxels];

constexpr int kNoAllocMaxDevices = 64;
float4* g_noalloc_ptr[kNoAllocMaxDevices] = {};
std::mutex g_noalloc_mutex;

// Device address of the built-in scratch on the CURRENT device.  In host code the array's
// name is only a stand-in; the address a kernel can use comes from cudaGetSymbolAddress,
// asked once per device with that device current.
int noalloc_scratch(float4** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (dev < 0 || dev >= kNoAllocMaxDevices)
        return fail(B200PROJ_ERR_LIMIT, "device ordinal %d is beyond the %d devices the allocation-free entry point tracks", dev, kNoAllocMaxDevices);
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (g_noalloc_ptr[dev] == nullptr) {
        float4* ptr = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, g_noalloc_accum);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress");
        g_noalloc_ptr[dev] = ptr;
    }
    *out = g_noalloc_ptr[dev];
    return B200PROJ_OK;
}

}  // namespace

extern "C" {

int b200proj_version(void) { return 300; }

#ifndef B200PROJ_SOURCE_STAMP
#define B200PROJ_SOURCE_STAMP ""
#endif
const char* b200proj_source_stamp(void) { return B200PROJ_SOURCE_STAMP; }

const char* b200proj_last_error(void) { return g_error; }

size_t b200proj_backproject_workspace_bytes(int dim, int64_t B, int64_t R, int64_t P, int64_t N,
                                           int interpolation, int has_weights) {
    if (!has_weights || (dim != 2 && dim != 3) || B < 1 || R < 2 || P < 1 || N < 2) return 0;
    const double voxels = (double)B * (dim == 3 ? R : 1) * R * (R / 2 + 1);
    const int t = interpolation == B200PROJ_CUBIC ? 4 : 2;
    const double taps = (double)B * P * N * (N / 2 + 1) * (dim == 3 ? t * t * t : t * t);
    // worth it once the scatter outweighs the two extra passes over the volume
    if (taps < 4.0 * voxels) return 0;
    if (dim == 3 && slab_plan(R, true).slabs > 1) return 0;      // beyond-L2 volumes take the slab-ordered path
    const double one = voxels * (double)sizeof(float4);
    return (size_t)one * (size_t)workspace_replicas(one, P);       // small reconstructions: several copies
}

int64_t b200proj_rec_boxsize(int64_t N, double oversampling) {
    const int64_t raw = (int64_t)std::ceil((double)N * oversampling);
    return raw + (raw % 2);
}

int b200proj_debug_index(int which, int R, int coordinate, int mirrored_in, int* mirrored_out) {
    SliceGeom g{};
    g.R = R; g.Rh = R / 2 + 1; g.half = R / 2;
    bool m = mirrored_in != 0;
    int r = INT_MIN;
    switch (which) {
        case 0: r = gather_col<false>(g, coordinate, m); break;
        case 1: r = gather_col<true>(g, coordinate, m); break;
        case 2: r = gather_line<false>(g, coordinate, m); break;
        case 3: r = gather_line<true>(g, coordinate, m); break;
        case 4: r = scatter_col(g, coordinate, m); break;
        case 5: r = scatter_line(g, coordinate, m); break;
        default: break;
    }
    if (mirrored_out != nullptr) *mirrored_out = m ? 1 : 0;
    return r;
}

int b200proj_project_2d_forw(const float* rec, int64_t B, int64_t R, const float* rot, int64_t B_rot,
                             const float* shifts, int64_t B_shift, int64_t P, int64_t N,
                             int interpolation, double oversampling, double cutoff, float* out,
                             void* stream) {
    return project_forw<2>(rec, B, R, rot, B_rot, shifts, B_shift, P, N, interpolation, oversampling, cutoff, out, nullptr, stream);
}
int b200proj_project_3d_to_2d_forw(const float* rec, int64_t B, int64_t R, const float* rot,
                                   int64_t B_rot, const float* shifts, int64_t B_shift, int64_t P,
                                   int64_t N, int interpolation, double oversampling, double cutoff,
                                   float* out, const int32_t* pose_order, void* stream) {
    return project_forw<3>(rec, B, R, rot, B_rot, shifts, B_shift, P, N, interpolation, oversampling, cutoff, out, pose_order, stream);
}

int b200proj_project_2d_back(const float* grad_proj, const float* rec, int64_t B, int64_t R,
                             const float* rot, int64_t B_rot, const float* shifts, int64_t B_shift,
                             int64_t P, int64_t N, int interpolation, double oversampling,
                             double cutoff, float* grad_rec, float* grad_rot, float* grad_shifts,
                             void* stream) {
    return project_back<2>(grad_proj, rec, B, R, rot, B_rot, shifts, B_shift, P, N, interpolation, oversampling, cutoff, grad_rec, grad_rot, grad_shifts, nullptr, stream);
}
int b200proj_project_3d_to_2d_back(const float* grad_proj, const float* rec, int64_t B, int64_t R,
                                   const float* rot, int64_t B_rot, const float* shifts,
                                   int64_t B_shift, int64_t P, int64_t N, int interpolation,
                                   double oversampling, double cutoff, float* grad_rec,
                                   float* grad_rot, float* grad_shifts, const int32_t* pose_order,
                                   void* stream) {
    return project_back<3>(grad_proj, rec, B, R, rot, B_rot, shifts, B_shift, P, N, interpolation, oversampling, cutoff, grad_rec, grad_rot, grad_shifts, pose_order, stream);
}

int b200proj_project_2d_forw_saving(const float* rec, int64_t B, int64_t R, const float* rot,
                                    int64_t B_rot, const float* shifts, int64_t B_shift, int64_t P,
                                    int64_t N, int interpolation, double oversampling, double cutoff,
                                    float* out, float* derivatives, void* stream) {
    return project_forw_saving<2>(rec, B, R, rot, B_rot, shifts, B_shift, P, N, interpolation, oversampling, cutoff, out, derivatives, nullptr, stream);
}
int b200proj_project_3d_to_2d_forw_saving(const float* rec, int64_t B, int64_t R, const float* rot,
                                          int64_t B_rot, const float* shifts, int64_t B_shift, int64_t P,
                                          int64_t N, int interpolation, double oversampling, double cutoff,
                                          float* out, float* derivatives, const int32_t* pose_order, void* stream) {
    return project_forw_saving<3>(rec, B, R, rot, B_rot, shifts, B_shift, P, N, interpolation, oversampling, cutoff, out, derivatives, pose_order, stream);
}
int b200proj_project_2d_back_saved(const float* grad_proj, const float* out, const float* derivatives,
                                   int64_t B, int64_t R, const float* rot, int64_t B_rot,
                                   const float* shifts, int64_t B_shift, int64_t P, int64_t N,
                                   int interpolation, double oversampling, double cutoff,
                                   float* grad_rec, float* grad_rot, float* grad_shifts, void* stream) {
    return project_back_saved<2>(grad_proj, out, derivatives, B, R, rot, B_rot, shifts, B_shift, P, N, interpolation, oversampling, cutoff, grad_rec, grad_rot, grad_shifts, nullptr, stream);
}
int b200proj_project_3d_to_2d_back_saved(const float* grad_proj, const float* out, const float* derivatives,
                                         int64_t B, int64_t R, const float* rot, int64_t B_rot,
                                         const float* shifts, int64_t B_shift, int64_t P, int64_t N,
                                         int interpolation, double oversampling, double cutoff,
                                         float* grad_rec, float* grad_rot, float* grad_shifts,
                                         const int32_t* pose_order, void* stream) {
    return project_back_saved<3>(grad_proj, out, derivatives, B, R, rot, B_rot, shifts, B_shift, P, N, interpolation, oversampling, cutoff, grad_rec, grad_rot, grad_shifts, pose_order, stream);
}

int b200proj_backproject_2d_forw(const float* proj, const float* weights, int64_t B, int64_t R,
                                 const float* rot, int64_t B_rot, const float* shifts,
                                 int64_t B_shift, int64_t P, int64_t N, int interpolation,
                                 double oversampling, double cutoff, float* data_rec,
                                 float* weight_rec, int accumulate, void* workspace, size_t workspace_bytes, void* stream) {
    return backproject_forw<2>(proj, weights, B, R, rot, B_rot, shifts, B_shift, P, N, interpolation, oversampling, cutoff, data_rec, weight_rec, accumulate, workspace, workspace_bytes, stream);
}
int b200proj_backproject_2d_to_3d_forw(const float* proj, const float* weights, int64_t B,
                                       int64_t R, const float* rot, int64_t B_rot,
                                       const float* shifts, int64_t B_shift, int64_t P, int64_t N,
                                       int interpolation, double oversampling, double cutoff,
                                       float* data_rec, float* weight_rec, int accumulate,                                        void* workspace, size_t workspace_bytes, void* stream) {
    return backproject_forw<3>(proj, weights, B, R, rot, B_rot, shifts, B_shift, P, N, interpolation, oversampling, cutoff, data_rec, weight_rec, accumulate, workspace, workspace_bytes, stream);
}

int b200proj_backproject_2d_back(const float* grad_data_rec, const float* grad_weight_rec,
                                 const float* proj, int64_t B, int64_t R, const float* rot,
                                 int64_t B_rot, const float* shifts, int64_t B_shift, int64_t P,
                                 int64_t N, int interpolation, double oversampling, double cutoff,
                                 float* grad_proj, float* grad_weights, float* grad_rot,
                                 float* grad_shifts, void* stream) {
    return backproject_back<2>(grad_data_rec, grad_weight_rec, proj, B, R, rot, B_rot, shifts, B_shift, P, N, interpolation, oversampling, cutoff, grad_proj, grad_weights, grad_rot, grad_shifts, nullptr, stream);
}
int b200proj_backproject_2d_to_3d_back(const float* grad_data_rec, const float* grad_weight_rec,
                                       const float* proj, int64_t B, int64_t R, const float* rot,
                                       int64_t B_rot, const float* shifts, int64_t B_shift,
                                       int64_t P, int64_t N, int interpolation,
                                       double oversampling, double cutoff, float* grad_proj,
                                       float* grad_weights, float* grad_rot, float* grad_shifts,
                                       const int32_t* pose_order, void* stream) {
    return backproject_back<3>(grad_data_rec, grad_weight_rec, proj, B, R, rot, B_rot, shifts, B_shift, P, N, interpolation, oversampling, cutoff, grad_proj, grad_weights, grad_rot, grad_shifts, pose_order, stream);
}

// ---- complex128 / float64 variants (same kernels instantiated for double) ----------------
int b200proj_project_2d_forw_f64(const double* rec, int64_t B, int64_t R, const double* rot, int64_t B_rot,
                             const double* shifts, int64_t B_shift, int64_t P, int64_t N,
                             int interpolation, double oversampling, double cutoff, double* out,
                             void* stream) {
    return project_forw<2>(rec, B, R, rot, B_rot, shifts, B_shift, P, N, interpolation, oversampling, cutoff, out, nullptr, stream);
}
int b200proj_project_3d_to_2d_forw_f64(const double* rec, int64_t B, int64_t R, const double* rot,
                                   int64_t B_rot, const double* shifts, int64_t B_shift, int64_t P,
                                   int64_t N, int interpolation, double oversampling, double cutoff,
                                   double* out, const int32_t* pose_order, void* stream) {
    return project_forw<3>(rec, B, R, rot, B_rot, shifts, B_shift, P, N, interpolation, oversampling, cutoff, out, pose_order, stream);
}

int b200proj_project_2d_back_f64(const double* grad_proj, const double* rec, int64_t B, int64_t R,
                             const double* rot, int64_t B_rot, const double* shifts, int64_t B_shift,
                             int64_t P, int64_t N, int interpolation, double oversampling,
                             double cutoff, double* grad_rec, double* grad_rot, double* grad_shifts,
                             void* stream) {
    return project_back<2>(grad_proj, rec, B, R, rot, B_rot, shifts, B_shift, P, N, interpolation, oversampling, cutoff, grad_rec, grad_rot, grad_shifts, nullptr, stream);
}
int b200proj_project_3d_to_2d_back_f64(const double* grad_proj, const double* rec, int64_t B, int64_t R,
                                   const double* rot, int64_t B_rot, const double* shifts,
                                   int64_t B_shift, int64_t P, int64_t N, int interpolation,
                                   double oversampling, double cutoff, double* grad_rec,
                                   double* grad_rot, double* grad_shifts, const int32_t* pose_order,
                                   void* stream) {
    return project_back<3>(grad_proj, rec, B, R, rot, B_rot, shifts, B_shift, P, N, interpolation, oversampling, cutoff, grad_rec, grad_rot, grad_shifts, pose_order, stream);
}

int b200proj_backproject_2d_forw_f64(const double* proj, const double* weights, int64_t B, int64_t R,
                                 const double* rot, int64_t B_rot, const double* shifts,
                                 int64_t B_shift, int64_t P, int64_t N, int interpolation,
                                 double oversampling, double cutoff, double* data_rec,
                                 double* weight_rec, int accumulate, void* workspace, size_t workspace_bytes, void* stream) {
    return backproject_forw<2>(proj, weights, B, R, rot, B_rot, shifts, B_shift, P, N, interpolation, oversampling, cutoff, data_rec, weight_rec, accumulate, workspace, workspace_bytes, stream);
}
int b200proj_backproject_2d_to_3d_forw_f64(const double* proj, const double* weights, int64_t B,
                                       int64_t R, const double* rot, int64_t B_rot,
                                       const double* shifts, int64_t B_shift, int64_t P, int64_t N,
                                       int interpolation, double oversampling, double cutoff,
                                       double* data_rec, double* weight_rec, int accumulate,                                        void* workspace, size_t workspace_bytes, void* stream) {
    return backproject_forw<3>(proj, weights, B, R, rot, B_rot, shifts, B_shift, P, N, interpolation, oversampling, cutoff, data_rec, weight_rec, accumulate, workspace, workspace_bytes, stream);
}

int b200proj_backproject_2d_back_f64(const double* grad_data_rec, const double* grad_weight_rec,
                                 const double* proj, int64_t B, int64_t R, const double* rot,
                                 int64_t B_rot, const double* shifts, int64_t B_shift, int64_t P,
                                 int64_t N, int interpolation, double oversampling, double cutoff,
                                 double* grad_proj, double* grad_weights, double* grad_rot,
                                 double* grad_shifts, void* stream) {
    return backproject_back<2>(grad_data_rec, grad_weight_rec, proj, B, R, rot, B_rot, shifts, B_shift, P, N, interpolation, oversampling, cutoff, grad_proj, grad_weights, grad_rot, grad_shifts, nullptr, stream);
}
int b200proj_backproject_2d_to_3d_back_f64(const double* grad_data_rec, const double* grad_weight_rec,
                                       const double* proj, int64_t B, int64_t R, const double* rot,
                                       int64_t B_rot, const double* shifts, int64_t B_shift,
                                       int64_t P, int64_t N, int interpolation,
                                       double oversampling, double cutoff, double* grad_proj,
                                       double* grad_weights, double* grad_rot, double* grad_shifts,
                                       const int32_t* pose_order, void* stream) {
    return backproject_back<3>(grad_data_rec, grad_weight_rec, proj, B, R, rot, B_rot, shifts, B_shift, P, N, interpolation, oversampling, cutoff, grad_proj, grad_weights, grad_rot, grad_shifts, pose_order, stream);
}

int b200proj_backproject_2d_to_3d_accumulate(const float* proj, const float* weights, int64_t B,
                                             int64_t R, const float* rot, int64_t B_rot,
                                             const float* shifts, int64_t B_shift, int64_t P,
                                             int64_t N, int interpolation, double oversampling,
                                             double cutoff, void* accumulator, void* stream) {
    return backproject_accumulate(proj, weights, B, R, rot, B_rot, shifts, B_shift, P, N, interpolation, oversampling, cutoff, accumulator, 0, -1, stream);
}

int b200proj_backproject_2d_to_3d_accumulate_slabs(const float* proj, const float* weights, int64_t B,
                                                   int64_t R, const float* rot, int64_t B_rot,
                                                   const float* shifts, int64_t B_shift, int64_t P,
                                                   int64_t N, int interpolation, double oversampling,
                                                   double cutoff, void* accumulator, int slab_first,
                                                   int slab_count, void* stream) {
    if (slab_count < 0) return fail(B200PROJ_ERR_ARGUMENT, "slab_count must be >= 1");
    return backproject_accumulate(proj, weights, B, R, rot, B_rot, shifts, B_shift, P, N, interpolation, oversampling, cutoff, accumulator, slab_first, slab_count, stream);
}

int b200proj_accumulator_slab_plan(int64_t R, int32_t* slabs, int32_t* planes_per_slab) {
    g_error[0] = 0;
    if (R < 2 || (R % 2) != 0 || slabs == nullptr || planes_per_slab == nullptr)
        return fail(B200PROJ_ERR_ARGUMENT, "need an even boxsize >= 2 and two output pointers");
    const SlabPlan plan = slab_plan(R, true, true);
    *slabs = plan.slabs;
    *planes_per_slab = plan.planes;
    return B200PROJ_OK;
}

int b200proj_accumulator_slab_voxels(int64_t R, int slab_first, int slab_count, int64_t first_voxel[2], int64_t voxel_count[2]) {
    g_error[0] = 0;
    if (R < 2 || (R % 2) != 0 || first_voxel == nullptr || voxel_count == nullptr)
        return fail(B200PROJ_ERR_ARGUMENT, "need an even boxsize >= 2 and two output arrays");
    const SlabPlan plan = slab_plan(R, true, true);
    if (slab_first < 0 || slab_count < 1 || slab_first + slab_count > plan.slabs)
        return fail(B200PROJ_ERR_ARGUMENT, "slabs [%d, %d) outside the plan of %d slabs", slab_first, slab_first + slab_count, plan.slabs);
    // signed plane coordinates [z_a, z_b) of the slabs; plane z is stored at index z < 0 ? z + R : z
    const int64_t half = R / 2, plane = R * (R / 2 + 1);
    const int64_t z_a = -half + 1 + (int64_t)slab_first * plan.planes;
    int64_t z_b = z_a + (int64_t)slab_count * plan.planes;
    if (z_b > half + 1) z_b = half + 1;
    const int64_t neg_b = z_b < 0 ? z_b : 0, pos_a = z_a > 0 ? z_a : 0;
    first_voxel[0] = (z_a < neg_b) ? (z_a + R) * plane : 0;            // planes with negative coordinates
    voxel_count[0] = (z_a < neg_b) ? (neg_b - z_a) * plane : 0;
    first_voxel[1] = (pos_a < z_b) ? pos_a * plane : 0;                // planes with coordinates >= 0
    voxel_count[1] = (pos_a < z_b) ? (z_b - pos_a) * plane : 0;
    return B200PROJ_OK;
}

size_t b200proj_accumulator_bytes(int64_t B, int64_t R) {
    if (B < 1 || R < 2) return 0;
    return (size_t)B * (size_t)R * (size_t)R * (size_t)(R / 2 + 1) * sizeof(float4);
}

int b200proj_accumulator_fold_range(const void* accumulator, int64_t first_voxel, int64_t voxel_count,
                                    float* data_rec, float* weight_rec, int accumulate, void* stream) {
    g_error[0] = 0;
    if (accumulator == nullptr || data_rec == nullptr || weight_rec == nullptr)
        return fail(B200PROJ_ERR_ARGUMENT, "accumulator, data_reconstruction and weight_reconstruction are all required");
    if (first_voxel < 0 || voxel_count < 0) return fail(B200PROJ_ERR_ARGUMENT, "voxel range must be non-negative (first=%lld, count=%lld)", (long long)first_voxel, (long long)voxel_count);
    if (voxel_count == 0) return B200PROJ_OK;
    const size_t n = (size_t)voxel_count;
    const size_t blocks = (n + 255) / 256;
    fold_interleaved_kernel<<<(unsigned)(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0, (cudaStream_t)stream>>>(
        (const float4*)accumulator + first_voxel, (float2*)data_rec + first_voxel, weight_rec + first_voxel, n, accumulate != 0);
    return check_launch("fold_interleaved launch");
}

int b200proj_accumulator_fold_normalized(const void* accumulator, int64_t first_voxel, int64_t voxel_count,
                                         double eps, float* normalized, void* stream) {
    g_error[0] = 0;
    if (accumulator == nullptr || normalized == nullptr) return fail(B200PROJ_ERR_ARGUMENT, "accumulator and output are required");
    if (first_voxel < 0 || voxel_count < 0) return fail(B200PROJ_ERR_ARGUMENT, "voxel range must be non-negative (first=%lld, count=%lld)", (long long)first_voxel, (long long)voxel_count);
    if (!(eps > 0.0)) return fail(B200PROJ_ERR_ARGUMENT, "eps must be positive");
    if (voxel_count == 0) return B200PROJ_OK;
    const size_t n = (size_t)voxel_count;
    const size_t blocks = (n + 255) / 256;
    fold_normalized_kernel<<<(unsigned)(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0, (cudaStream_t)stream>>>(
        (const float4*)accumulator + first_voxel, (float2*)normalized + first_voxel, n, (float)eps);
    return check_launch("fold_normalized launch");
}

int64_t b200proj_cutoff_pack_index(int64_t N, double cutoff, int32_t* index) {
    g_error[0] = 0;
    if (N < 2 || (N % 2) != 0 || N > 2048 || std::isnan(cutoff)) { fail(B200PROJ_ERR_ARGUMENT, "need an even projection boxsize in [2, 2048] and a cutoff"); return -1; }
    // the kernels' own test (pixel_setup): kr*kr + kc*kc > float(cutoff)^2 in fp32 excludes a pixel
    const float rc = (float)cutoff, cutoff_sq = rc * rc;
    const int64_t Nh = N / 2 + 1;
    int64_t count = 0;
    for (int64_t i = 0; i < N; ++i) {
        const float kr = (float)((i <= N / 2) ? i : i - N);
        for (int64_t j = 0; j < Nh; ++j) {
            const float kc = (float)j;
            const bool inside = !(kr * kr + kc * kc > cutoff_sq);
            if (index != nullptr) index[i * Nh + j] = inside ? (int32_t)count : -1;
            count += inside ? 1 : 0;
        }
    }
    return count;
}

int b200proj_project_3d_to_2d_forw_packed(const float* rec, int64_t B, int64_t R, const float* rot,
                                          int64_t B_rot, const float* shifts, int64_t B_shift, int64_t P,
                                          int64_t N, int interpolation, double oversampling, double cutoff,
                                          float* out_packed, const int32_t* pack_index, int64_t pack_count,
                                          const int32_t* pose_order, void* stream) {
    Launch L;
    if (int rc = prepare(L, 3, B, R, B_rot, rot, shifts, B_shift, P, N, interpolation, oversampling, cutoff)) return rc;
    if (rec == nullptr || out_packed == nullptr || pack_index == nullptr)
        return fail(B200PROJ_ERR_ARGUMENT, "reconstruction / output / pack_index pointer is NULL");
    if (pack_count != b200proj_cutoff_pack_index(N, cutoff, nullptr))
        return fail(B200PROJ_ERR_ARGUMENT, "pack_count %lld is not the number of pixels inside the cutoff (%lld)",
                    (long long)pack_count, (long long)b200proj_cutoff_pack_index(N, cutoff, nullptr));
    L.g.order = pose_order;
    L.g.pack_index = pack_index;
    L.g.pack_count = (int)pack_count;
    if (P == 0 || pack_count == 0) return B200PROJ_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (interpolation == B200PROJ_CUBIC)
        project_forw_kernel<3, true, float, true><<<L.grid, kBlockThreads, 0, s>>>((const float2*)rec, rot, shifts, (float2*)out_packed, L.g);
    else
        project_forw_kernel<3, false, float, true><<<L.grid, kBlockThreads, 0, s>>>((const float2*)rec, rot, shifts, (float2*)out_packed, L.g);
    return check_launch("project_forw (packed) launch");
}

int b200proj_reduction_rate_probe(int pattern, float* buffer, size_t buffer_bytes, int blocks, int iterations, void* stream) {
    g_error[0] = 0;
    if (buffer == nullptr || (reinterpret_cast<uintptr_t>(buffer) & 15u) != 0) return fail(B200PROJ_ERR_ARGUMENT, "buffer must be a 16-byte aligned device pointer");
    if (pattern < 0 || pattern > 5 || blocks < 1 || iterations < 1) return fail(B200PROJ_ERR_ARGUMENT, "pattern must be 0..5, blocks and iterations >= 1");
    const size_t unit = pattern <= 2 ? 16 : 8;
    const size_t units = buffer_bytes / unit;
    if (units < 16 || units > 0xffffffffull) return fail(B200PROJ_ERR_LIMIT, "buffer of %zu bytes holds too few or too many units", buffer_bytes);
    cudaStream_t s = (cudaStream_t)stream;
    switch (pattern) {
        case 0: reduction_rate_kernel<0><<<blocks, 256, 0, s>>>(buffer, (unsigned)units, iterations); break;
        case 1: reduction_rate_kernel<1><<<blocks, 256, 0, s>>>(buffer, (unsigned)units, iterations); break;
        case 2: reduction_rate_kernel<2><<<blocks, 256, 0, s>>>(buffer, (unsigned)units, iterations); break;
        case 3: reduction_rate_kernel<3><<<blocks, 256, 0, s>>>(buffer, (unsigned)units, iterations); break;
        case 4: reduction_rate_kernel<4><<<blocks, 256, 0, s>>>(buffer, (unsigned)units, iterations); break;
        default: reduction_rate_kernel<5><<<blocks, 256, 0, s>>>(buffer, (unsigned)units, iterations); break;
    }
    return check_launch("reduction_rate_probe launch");
}

int b200proj_reduction_rate_probe_streaming(float* target, size_t target_bytes, size_t window_bytes,
                                            const float* source, size_t source_bytes, int blocks,
                                            int iterations, int evict_last, void* stream) {
    g_error[0] = 0;
    if (target == nullptr || (reinterpret_cast<uintptr_t>(target) & 15u) != 0 || source == nullptr || (reinterpret_cast<uintptr_t>(source) & 7u) != 0)
        return fail(B200PROJ_ERR_ARGUMENT, "target must be a 16-byte and source an 8-byte aligned device pointer");
    if (blocks < 1 || iterations < 1) return fail(B200PROJ_ERR_ARGUMENT, "blocks and iterations must be >= 1");
    const size_t units = target_bytes / 16, window = window_bytes / 16, src_units = source_bytes / 8;
    if (window < 16 || units < window || units > 0xffffffffull || src_units < 256 || src_units > 0xffffffffull)
        return fail(B200PROJ_ERR_LIMIT, "target of %zu bytes, window of %zu bytes or source of %zu bytes out of range", target_bytes, window_bytes, source_bytes);
    if (evict_last)
        reduction_stream_kernel<true><<<blocks, 256, 0, (cudaStream_t)stream>>>(target, (unsigned)units, (unsigned)window,
                                                                               reinterpret_cast<const float2*>(source), (unsigned)src_units, iterations);
    else
        reduction_stream_kernel<false><<<blocks, 256, 0, (cudaStream_t)stream>>>(target, (unsigned)units, (unsigned)window,
                                                                                reinterpret_cast<const float2*>(source), (unsigned)src_units, iterations);
    return check_launch("reduction_rate_probe_streaming launch");
}

int b200proj_accumulator_fold(const void* accumulator, int64_t B, int64_t R, float* data_rec,
                              float* weight_rec, int accumulate, void* stream) {
    if (B < 1 || R < 2 || (R % 2) != 0) return fail(B200PROJ_ERR_ARGUMENT, "batch size must be >= 1 and the boxsize even (B=%lld, R=%lld)", (long long)B, (long long)R);
    return b200proj_accumulator_fold_range(accumulator, 0, B * R * R * (R / 2 + 1), data_rec, weight_rec, accumulate, stream);
}

int b200proj_pad_fftshift(const float* real, int64_t batch, int dims, int64_t n, int64_t m, float* out, void* stream) {
    return pad_shift(real, batch, dims, n, m, 1, out, stream);
}
int b200proj_pad_fftshift_f64(const double* real, int64_t batch, int dims, int64_t n, int64_t m, double* out, void* stream) {
    return pad_shift(real, batch, dims, n, m, 1, out, stream);
}
int b200proj_ifftshift_crop(const float* full, int64_t batch, int dims, int64_t m, int64_t n, float* out, void* stream) {
    return pad_shift(full, batch, dims, n, m, 0, out, stream);
}
int b200proj_ifftshift_crop_f64(const double* full, int64_t batch, int dims, int64_t m, int64_t n, double* out, void* stream) {
    return pad_shift(full, batch, dims, n, m, 0, out, stream);
}

int b200proj_pose_order_3d(const float* rot, int64_t B, int64_t B_rot, int64_t P, int32_t* order, void* stream) {
    return pose_order_3d(rot, B, B_rot, P, order, stream);
}
int b200proj_pose_order_3d_f64(const double* rot, int64_t B, int64_t B_rot, int64_t P, int32_t* order, void* stream) {
    return pose_order_3d(rot, B, B_rot, P, order, stream);
}

int b200proj_backproject_2d_to_3d_forw_noalloc(const float* proj, const float* weights, int64_t B,
                                               int64_t R, const float* rot, int64_t B_rot,
                                               const float* shifts, int64_t B_shift, int64_t P,
                                               int64_t N, int interpolation, double oversampling,
                                               double cutoff, float* data_rec, float* weight_rec,
                                               int accumulate, void* stream) {
    Launch L;
    if (int rc = prepare(L, 3, B, R, B_rot, rot, shifts, B_shift, P, N, interpolation, oversampling, cutoff)) return rc;
    if (proj == nullptr || weights == nullptr || data_rec == nullptr || weight_rec == nullptr)
        return fail(B200PROJ_ERR_ARGUMENT, "projections, weights, data_reconstruction and weight_reconstruction are all required");
    if (R != b200proj_rec_boxsize(N, oversampling))
        return fail(B200PROJ_ERR_ARGUMENT, "reconstruction boxsize %lld does not match ceil(N*oversampling) rounded up to even = %lld",
                    (long long)R, (long long)b200proj_rec_boxsize(N, oversampling));
    if ((long long)L.rec_count > kNoAllocMaxVoxels)
        return fail(B200PROJ_ERR_LIMIT, "B*R*R*(R/2+1) = %lld voxels exceed the built-in scratch of %lld voxels (box 64, one batch item); "
                    "use b200proj_backproject_2d_to_3d_forw with a caller-provided workspace",
                    (long long)L.rec_count, kNoAllocMaxVoxels);
    float4* acc = nullptr;
    if (int rc = noalloc_scratch(&acc)) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    // the scratch keeps the previous call's sums: clear the part this call uses
    if (int rc = zero_async(acc, L.rec_count * sizeof(float4), s)) return rc;
    if (P > 0) {
        if (interpolation == B200PROJ_CUBIC)
            backproject_forw_interleaved_kernel<3, true><<<L.grid, kBlockThreads, 0, s>>>((const float2*)proj, weights, rot, shifts, acc, L.g);
        else
            backproject_forw_interleaved_kernel<3, false><<<L.grid, kBlockThreads, 0, s>>>((const float2*)proj, weights, rot, shifts, acc, L.g);
        if (int rc = check_launch("backproject_forw (built-in scratch) launch")) return rc;
    }
    const size_t blocks = (L.rec_count + 255) / 256;
    fold_interleaved_kernel<<<(unsigned)(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0, s>>>(acc, (float2*)data_rec, weight_rec, L.rec_count, accumulate != 0);
    return check_launch("fold_interleaved launch");
}

}  // extern "C"
