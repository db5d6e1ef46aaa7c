// The four kernel families of the Fourier-slice operators, each templated on the
// dimensionality (2: image -> image, 3: volume -> slice) and the interpolation.
//
//   project_forw_kernel      gather   rec -> projections            (forward projection)
//   project_back_kernel      scatter  grad_proj -> grad_rec, + pose gradients
//   backproject_forw_kernel  scatter  projections (+weights) -> data / weight volumes
//   backproject_back_kernel  gather   grad volumes -> grad_proj / grad_weights, + pose grads
//
// One block handles one 16x16 tile of one slice (pose p of batch item b); blockIdx.x
// enumerates (b, p, tile).  No kernel waits on another block, so none can hang.
#pragma once

#include "fourier_slice_device.cuh"

namespace b200proj {

struct BlockWork {
    int b, p, i, j;
    bool in_image;
    size_t pix;     // element offset of (b, p, i, j) in a [B, P, N, Nh] tensor
};

__device__ __forceinline__ BlockWork block_work(const SliceGeom& g) {
    BlockWork w;
    const int tiles = g.tiles_j * g.tiles_i;
    const int bp = blockIdx.x / tiles;
    const int tile = blockIdx.x - bp * tiles;
    w.b = bp / g.P;
    w.p = bp - w.b * g.P;
    tile_pixel(g, tile, w.i, w.j);
    w.in_image = w.i < g.N && w.j < g.Nh;
    w.pix = ((size_t)bp * (size_t)g.N + (size_t)w.i) * (size_t)g.Nh + (size_t)w.j;
    return w;
}

template <int DIM>
__device__ __forceinline__ const float* pose_rot(const SliceGeom& g, const float* rot, int b, int p) {
    return rot + (size_t)b * g.rot_stride_b + (size_t)p * (DIM * DIM);
}
__device__ __forceinline__ const float* pose_shift(const SliceGeom& g, const float* shifts, int b, int p) {
    return shifts + (size_t)b * g.shift_stride_b + (size_t)p * 2;
}

// ---- forward projection -----------------------------------------------------------------
// reference semantics: csrc/cpu/3d/projection_3d_to_2d_kernels.cpp:155-207
template <int DIM, bool CUBIC>
__global__ void __launch_bounds__(kBlockThreads)
project_forw_kernel(const float2* __restrict__ rec, const float* __restrict__ rot,
                    const float* __restrict__ shifts, float2* __restrict__ out, const SliceGeom g) {
    const BlockWork w = block_work(g);
    Pixel px;
    px.c = px.r = px.d = 0.f;
    const bool valid = w.in_image && pixel_setup<DIM>(g, pose_rot<DIM>(g, rot, w.b, w.p), w.i, w.j, px);
    float2 v, gc, gr, gd;
    // all 32 lanes take part: the lanes of a group fetch each other's taps
    interpolate_coop<DIM, CUBIC, false>(g, rec + (size_t)w.b * g.vol_elems, px, valid, v, gc, gr, gd);
    if (!w.in_image) return;
    if (valid && g.has_shift) {
        const float* s = pose_shift(g, shifts, w.b, w.p);
        v = cmul(v, phase_ramp(g, px, __ldg(s), __ldg(s + 1)));
    }
    // streaming store: the projections are written once and never re-read by this kernel,
    // keep the cache for the volume
    __stcs(out + w.pix, v);
}

// Pose-gradient terms shared by the two backward kernels.
//   rotation:  dL/dR[a][m] += s_m * Re(u * conj(grad_a)),  a: (c, r, d) rows, s = (sc, sr, 0)
//   shift:     dL/ds[n]    += q_n * (u.y * val.x - u.x * val.y),  q = -2*pi*k_n/N
template <int DIM, bool NEED_ROT, bool NEED_SHIFT>
__device__ __forceinline__ void pose_grad_terms(const SliceGeom& g, const Pixel& px, float2 u_rot,
                                                float2 u_shift, float2 val_shift, float2 g_c,
                                                float2 g_r, float2 g_d,
                                                float (&acc)[2 * DIM + 2]) {
    if (NEED_ROT) {
        const float dc = u_rot.x * g_c.x + u_rot.y * g_c.y;
        const float dr = u_rot.x * g_r.x + u_rot.y * g_r.y;
        acc[0] += dc * px.sc;
        acc[1] += dc * px.sr;
        acc[2] += dr * px.sc;
        acc[3] += dr * px.sr;
        if (DIM == 3) {
            const float dd = u_rot.x * g_d.x + u_rot.y * g_d.y;
            acc[4] += dd * px.sc;
            acc[5] += dd * px.sr;
        }
    }
    if (NEED_SHIFT) {
        const float cross = u_shift.y * val_shift.x - u_shift.x * val_shift.y;
        acc[2 * DIM + 0] += (float)(g.shift_scale * (double)px.kr) * cross;
        acc[2 * DIM + 1] += (float)(g.shift_scale * (double)px.kc) * cross;
    }
}

template <int DIM>
__device__ __forceinline__ void pose_grad_flush(const SliceGeom& g, float (&acc)[2 * DIM + 2],
                                                float* grad_rot, float* grad_shift, int b, int p) {
    float* dst[2 * DIM + 2];
    float* gr = grad_rot ? grad_rot + (size_t)b * g.rot_stride_b + (size_t)p * (DIM * DIM) : nullptr;
    float* gs = grad_shift ? grad_shift + (size_t)b * g.shift_stride_b + (size_t)p * 2 : nullptr;
#pragma unroll
    for (int a = 0; a < DIM; ++a) {
        dst[2 * a + 0] = gr ? gr + a * DIM + 0 : nullptr;   // column 2 of a 3x3 gradient stays 0
        dst[2 * a + 1] = gr ? gr + a * DIM + 1 : nullptr;
    }
    dst[2 * DIM + 0] = gs;
    dst[2 * DIM + 1] = gs ? gs + 1 : nullptr;
    block_reduce_add<2 * DIM + 2>(acc, dst);
}

// ---- backward of forward projection -----------------------------------------------------
// reference semantics: csrc/cpu/3d/projection_3d_to_2d_kernels.cpp:283-396
template <int DIM, bool CUBIC, bool NEED_ROT, bool NEED_SHIFT>
__global__ void __launch_bounds__(kBlockThreads)
project_back_kernel(const float2* __restrict__ grad_proj, const float2* __restrict__ rec,
                    const float* __restrict__ rot, const float* __restrict__ shifts,
                    float2* __restrict__ grad_rec, float* __restrict__ grad_rot,
                    float* __restrict__ grad_shift, const SliceGeom g) {
    const BlockWork w = block_work(g);
    float acc[2 * DIM + 2];
#pragma unroll
    for (int q = 0; q < 2 * DIM + 2; ++q) acc[q] = 0.f;
    Pixel px;
    px.c = px.r = px.d = px.sc = px.sr = px.kr = px.kc = 0.f;
    const bool active = w.in_image &&
                        pixel_setup<DIM>(g, pose_rot<DIM>(g, rot, w.b, w.p), w.i, w.j, px) &&
                        !(w.j == 0 && w.i >= g.N / 2);
    float2 val = make_float2(0.f, 0.f), gc = val, gr = val, gd = val;
    if (NEED_ROT || NEED_SHIFT)      // cooperative gather: every lane of the warp takes part
        interpolate_coop<DIM, CUBIC, NEED_ROT>(g, rec + (size_t)w.b * g.vol_elems, px, active, val, gc, gr, gd);
    float2 orig = make_float2(0.f, 0.f), u = orig, ph = make_float2(1.f, 0.f);
    if (active) {
        orig = __ldcs(grad_proj + w.pix);
        u = orig;
        if (g.has_shift) {
            const float* s = pose_shift(g, shifts, w.b, w.p);
            ph = phase_ramp(g, px, __ldg(s), __ldg(s + 1));
            u = cmul_conj(orig, ph);
        }
    }
    // cooperative scatter: every lane of the warp takes part
    scatter_coop<DIM, CUBIC, false, false, false>(g, grad_rec + (size_t)w.b * g.vol_elems, nullptr, nullptr,
                                                  px, active, u, 0.f);
    if (active) {
        if (NEED_ROT || NEED_SHIFT) {
            const float2 mod = g.has_shift ? cmul(val, ph) : val;
            pose_grad_terms<DIM, NEED_ROT, NEED_SHIFT>(g, px, u, orig, mod, gc, gr, gd, acc);
        }
    }
    if (NEED_ROT || NEED_SHIFT) pose_grad_flush<DIM>(g, acc, grad_rot, grad_shift, w.b, w.p);
}

// ---- back-projection --------------------------------------------------------------------
// reference semantics: csrc/cpu/3d/backprojection_2d_to_3d_kernels.cpp:177-291
// Slice value with the conjugate shift ramp applied, and its weight (shared by both kernels).
template <int DIM, bool WEIGHTS>
__device__ __forceinline__ bool backproject_pixel(const SliceGeom& g, const BlockWork& w,
                                                  const float2* __restrict__ proj,
                                                  const float* __restrict__ weights,
                                                  const float* __restrict__ rot,
                                                  const float* __restrict__ shifts, Pixel& px,
                                                  float2& v, float& wv) {
    px.c = px.r = px.d = 0.f;
    v = make_float2(0.f, 0.f);
    wv = 0.f;
    const bool active = w.in_image && !(w.j == 0 && w.i >= g.N / 2) &&
                        pixel_setup<DIM>(g, pose_rot<DIM>(g, rot, w.b, w.p), w.i, w.j, px);
    if (active) {
        v = __ldcs(proj + w.pix);
        if (g.has_shift) {
            const float* s = pose_shift(g, shifts, w.b, w.p);
            v = cmul_conj(v, phase_ramp(g, px, __ldg(s), __ldg(s + 1)));
        }
        if (WEIGHTS) wv = __ldcs(weights + w.pix);
    }
    return active;
}

template <int DIM, bool CUBIC, bool WEIGHTS>
__global__ void __launch_bounds__(kBlockThreads)
backproject_forw_kernel(const float2* __restrict__ proj, const float* __restrict__ weights,
                        const float* __restrict__ rot, const float* __restrict__ shifts,
                        float2* __restrict__ data_rec, float* __restrict__ weight_rec,
                        const SliceGeom g) {
    const BlockWork w = block_work(g);
    Pixel px;
    float2 v;
    float wv;
    const bool active = backproject_pixel<DIM, WEIGHTS>(g, w, proj, weights, rot, shifts, px, v, wv);
    scatter_coop<DIM, CUBIC, WEIGHTS, true, false>(g, data_rec + (size_t)w.b * g.vol_elems,
                                                   WEIGHTS ? weight_rec + (size_t)w.b * g.vol_elems : nullptr,
                                                   nullptr, px, active, v, wv);
}

// Back-projection with weights into the interleaved accumulation volume (workspace), and
// the pass that folds it into the caller's data / weight volumes.
template <int DIM, bool CUBIC>
__global__ void __launch_bounds__(kBlockThreads)
backproject_forw_interleaved_kernel(const float2* __restrict__ proj, const float* __restrict__ weights,
                                    const float* __restrict__ rot, const float* __restrict__ shifts,
                                    float4* __restrict__ accum, const SliceGeom g) {
    const BlockWork w = block_work(g);
    Pixel px;
    float2 v;
    float wv;
    const bool active = backproject_pixel<DIM, true>(g, w, proj, weights, rot, shifts, px, v, wv);
    scatter_coop<DIM, CUBIC, true, true, true>(g, nullptr, nullptr, accum + (size_t)w.b * g.vol_elems,
                                               px, active, v, wv);
}

// data[k] (+)= accum[k].xy, weight[k] (+)= accum[k].z
__global__ void __launch_bounds__(256)
fold_interleaved_kernel(const float4* __restrict__ accum, float2* __restrict__ data,
                        float* __restrict__ weight, size_t n, int accumulate) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t k = (size_t)blockIdx.x * blockDim.x + threadIdx.x; k < n; k += stride) {
        const float4 a = __ldcs(accum + k);
        float2 d = make_float2(a.x, a.y);
        float wv = a.z;
        if (accumulate) {
            const float2 d0 = data[k];
            d.x += d0.x;
            d.y += d0.y;
            wv += weight[k];
        }
        data[k] = d;
        weight[k] = wv;
    }
}

// ---- backward of back-projection --------------------------------------------------------
// reference semantics: csrc/cpu/3d/backprojection_2d_to_3d_kernels.cpp:417-583
template <int DIM, bool CUBIC, bool NEED_ROT, bool NEED_SHIFT>
__global__ void __launch_bounds__(kBlockThreads)
backproject_back_kernel(const float2* __restrict__ grad_data_rec,
                        const float* __restrict__ grad_weight_rec,
                        const float2* __restrict__ proj, const float* __restrict__ rot,
                        const float* __restrict__ shifts, float2* __restrict__ grad_proj,
                        float* __restrict__ grad_weights, float* __restrict__ grad_rot,
                        float* __restrict__ grad_shift, const SliceGeom g) {
    const BlockWork w = block_work(g);
    float acc[2 * DIM + 2];
#pragma unroll
    for (int q = 0; q < 2 * DIM + 2; ++q) acc[q] = 0.f;
    Pixel px;
    px.c = px.r = px.d = px.sc = px.sr = px.kr = px.kc = 0.f;
    const bool active = w.in_image &&
                        pixel_setup<DIM>(g, pose_rot<DIM>(g, rot, w.b, w.p), w.i, w.j, px) &&
                        !(w.j == 0 && w.i >= g.N / 2);
    const bool write_w = grad_weight_rec != nullptr && grad_weights != nullptr;
    float2 raw, gc, gr, gd;
    // cooperative gather: every lane of the warp takes part
    interpolate_coop<DIM, CUBIC, NEED_ROT>(g, grad_data_rec + (size_t)w.b * g.vol_elems, px, active, raw, gc, gr, gd);
    if (active) {
        float2 ph = make_float2(1.f, 0.f);
        float2 v = raw;
        if (g.has_shift) {
            const float* s = pose_shift(g, shifts, w.b, w.p);
            ph = phase_ramp(g, px, __ldg(s), __ldg(s + 1));
            v = cmul(raw, ph);
        }
        __stcs(grad_proj + w.pix, v);
        if (write_w)
            __stcs(grad_weights + w.pix,
                   gather_weight_grad<DIM>(g, grad_weight_rec + (size_t)w.b * g.vol_elems, px));
        if (NEED_ROT || NEED_SHIFT) {
            float2 pv = __ldcs(proj + w.pix);
            if (g.has_shift) pv = cmul_conj(pv, ph);
            pose_grad_terms<DIM, NEED_ROT, NEED_SHIFT>(g, px, pv, pv, raw, gc, gr, gd, acc);
        }
    } else if (w.in_image) {
        __stcs(grad_proj + w.pix, make_float2(0.f, 0.f));
        if (write_w) __stcs(grad_weights + w.pix, 0.f);
    }
    if (NEED_ROT || NEED_SHIFT) pose_grad_flush<DIM>(g, acc, grad_rot, grad_shift, w.b, w.p);
}

}  // namespace b200proj
