// The four kernel families of the Fourier-slice operators, each templated on the
// dimensionality (2: image -> image, 3: volume -> slice) and the interpolation.
//
//   project_forw_kernel      gather   rec -> projections            (forward projection)
//   project_back_kernel      scatter  grad_proj -> grad_rec, + pose gradients
//   backproject_forw_kernel  scatter  projections (+weights) -> data / weight volumes
//   backproject_back_kernel  gather   grad volumes -> grad_proj / grad_weights, + pose grads
//
// One block handles one 16x16 tile of one slice (pose p of batch item b): blockIdx.x is the
// tile, (blockIdx.y, blockIdx.z) the slice.  No kernel waits on another block, so none can hang.
#pragma once

#include "fourier_slice_device.cuh"

namespace b200proj {

#ifndef PB_MIN_BLOCKS
#define PB_MIN_BLOCKS 4
#endif

struct BlockWork {
    int b, p, i, j;
    bool in_image;
    size_t pix;     // element offset of (b, p, i, j) in a [B, P, N, Nh] tensor
};

// Grid: x = tile of the slice, (y, z) = the slice.  Three decodings keep integer division out
// of the common cases (every thread decodes its block): one batch item: p = y + 32768*z;
// several batch items of at most 32768 poses: b = z, p = y; otherwise the flat slice index
// b*P + p = y + 32768*z is divided by P.
constexpr int kGridYBits = 15;

template <bool WIDE_PIX = false>
__device__ __forceinline__ BlockWork block_work(const SliceGeom& g) {
    BlockWork w;
    const int y = (int)blockIdx.y, z = (int)blockIdx.z;
    int b, p;
    if (g.decode == 0) {
        b = 0;
        p = y + (z << kGridYBits);
    } else if (g.decode == 1) {
        b = z;
        p = y;
    } else {
        const int bp = y + (z << kGridYBits);
        b = bp / g.P;
        p = bp - b * g.P;
    }
    int k = b * g.P + p;
    bool slice_ok = p < g.P && k < g.BP;
    if (g.order != nullptr && slice_ok) {
        // block k handles slice order[k], which lies in the same batch item; any other entry
        // (a malformed order) makes the block idle instead of reading out of bounds
        p = __ldg(g.order + k) - b * g.P;
        slice_ok = (unsigned)p < (unsigned)g.P;
    }
    if (!slice_ok) b = p = 0;
    w.b = b;
    w.p = p;
    tile_pixel(g, (int)blockIdx.x, w.i, w.j);
    w.in_image = w.i < g.N && w.j < g.Nh && slice_ok;
    // WIDE_PIX: the same offset as one 64-bit expression per thread.  It costs the cubic 3D
    // forward kernel 9 registers (57 instead of 48) and that is its purpose: the kernel is bound
    // by the L1TEX data pipe and runs slower with five resident blocks per SM than with four
    // (measured 4.44 vs 4.09 ms per 10,000 poses of the box-256 workload; a larger L1 carve-out,
    // taller blocks and plane-sorted slices did not change that).
    if (WIDE_PIX)
        w.pix = ((size_t)(b * g.P + p) * (size_t)g.N + (size_t)w.i) * (size_t)g.Nh + (size_t)w.j;
    else    // block-uniform slice base (64-bit) + 32-bit offset inside the slice
        w.pix = (size_t)(b * g.P + p) * (size_t)g.slice_pixels + (size_t)(w.i * g.Nh + w.j);
    return w;
}

template <int DIM, typename R>
__device__ __forceinline__ const R* pose_rot(const SliceGeom& g, const R* rot, int b, int p) {
    return rot + (size_t)b * g.rot_stride_b + (size_t)p * (DIM * DIM);
}
template <typename R>
__device__ __forceinline__ const R* pose_shift(const SliceGeom& g, const R* shifts, int b, int p) {
    return shifts + (size_t)b * g.shift_stride_b + (size_t)p * 2;
}

// ---- forward projection -----------------------------------------------------------------
// reference semantics: csrc/cpu/3d/projection_3d_to_2d_kernels.cpp:155-207
// PACKED: only the pixels inside the cutoff are written, side by side ([B, P, pack_count]; the
// position of a pixel comes from g.pack_index), for callers that copy the projections to the host
// and do not want to move the zeros outside the cutoff over PCIe.
template <int DIM, bool CUBIC, typename R, bool PACKED = false>
__global__ void __launch_bounds__(kBlockThreads)
project_forw_kernel(const C2<R>* __restrict__ rec, const R* __restrict__ rot,
                    const R* __restrict__ shifts, C2<R>* __restrict__ out, const SliceGeom g) {
    const BlockWork w = block_work<CUBIC && DIM == 3>(g);
    PixelT<R> px;
    px.c = px.r = px.d = 0.f;
    const bool valid = w.in_image && pixel_setup<DIM>(g, pose_rot<DIM>(g, rot, w.b, w.p), w.i, w.j, px);
    C2<R> v, gc, gr, gd;
    // all 32 lanes take part: the lanes of a group fetch each other's taps
    interpolate_any<DIM, CUBIC, false>(g, rec + (size_t)w.b * g.vol_elems, px, valid, v, gc, gr, gd);
    if (!w.in_image) return;
    if (valid && g.has_shift) {
        const R* s = pose_shift(g, shifts, w.b, w.p);
        v = cmul(v, phase_ramp(g, px, __ldg(s), __ldg(s + 1)));
    }
    // streaming store: the projections are written once and never re-read by this kernel,
    // keep the cache for the volume
    if constexpr (PACKED) {
        if (valid) {
            const int slot = __ldg(g.pack_index + (w.i * g.Nh + w.j));
            if (slot >= 0) __stcs(out + ((size_t)(w.b * g.P + w.p) * (size_t)g.pack_count + (size_t)slot), v);
        }
    } else {
        __stcs(out + w.pix, v);
    }
}

// Forward projection that also writes the derivatives of every output pixel with respect to its
// sample position (c, r, d), with the shift phase applied like the pixel itself: derivs is planar,
// [DIM][B, P, N, Nh].  The backward pass of a step that needs pose gradients then has nothing to
// gather (project_back_saved_kernel): the rotation gradient of a pixel is
// Re(grad * conj(derivative)) * sample frequency, the same numbers project_back_kernel forms from a
// second gather of the volume.  Pixels outside the cutoff are not written (and never read).
template <int DIM, bool CUBIC>
__global__ void __launch_bounds__(kBlockThreads)
project_forw_saving_kernel(const float2* __restrict__ rec, const float* __restrict__ rot,
                           const float* __restrict__ shifts, float2* __restrict__ out,
                           float2* __restrict__ derivs, const SliceGeom g) {
    const BlockWork w = block_work(g);
    Pixel px;
    px.c = px.r = px.d = 0.f;
    const bool valid = w.in_image && pixel_setup<DIM>(g, pose_rot<DIM>(g, rot, w.b, w.p), w.i, w.j, px);
    float2 v, gc, gr, gd;
    interpolate_any<DIM, CUBIC, true>(g, rec + (size_t)w.b * g.vol_elems, px, valid, v, gc, gr, gd);
    if (!w.in_image) return;
    if (valid && g.has_shift) {
        const float* s = pose_shift(g, shifts, w.b, w.p);
        const float2 ph = phase_ramp(g, px, __ldg(s), __ldg(s + 1));
        v = cmul(v, ph);
        gc = cmul(gc, ph);
        gr = cmul(gr, ph);
        if (DIM == 3) gd = cmul(gd, ph);
    }
    __stcs(out + w.pix, v);
    if (valid) {
        const size_t plane = (size_t)g.BP * (size_t)g.slice_pixels;
        __stcs(derivs + w.pix, gc);
        __stcs(derivs + plane + w.pix, gr);
        if (DIM == 3) __stcs(derivs + 2 * plane + w.pix, gd);
    }
}

// Linear interpolation, two pixels per lane: the 4- and 8-tap gathers are bound by instruction
// issue, and a good part of a pixel's instructions does not depend on its row (block decoding,
// pose loads, the column's share of the rotated position and of the shift phase).  Here a block
// covers 16 columns x 32 rows and every lane handles pixels (i, j) and (i + 16, j), forming those
// terms once.  The arithmetic per pixel is that of project_forw_kernel, operation for operation,
// so the outputs are bit-identical.
template <int DIM, typename R>
__global__ void __launch_bounds__(kBlockThreads)
project_forw_rows2_kernel(const C2<R>* __restrict__ rec, const R* __restrict__ rot,
                          const R* __restrict__ shifts, C2<R>* __restrict__ out, const SliceGeom g) {
    // slice of this block (same decodings as block_work)
    const int y = (int)blockIdx.y, z = (int)blockIdx.z;
    int b, p;
    if (g.decode == 0) { b = 0; p = y + (z << kGridYBits); }
    else if (g.decode == 1) { b = z; p = y; }
    else { const int bp = y + (z << kGridYBits); b = bp / g.P; p = bp - b * g.P; }
    bool slice_ok = p < g.P && b * g.P + p < g.BP;
    if (g.order != nullptr && slice_ok) {
        p = __ldg(g.order + (b * g.P + p)) - b * g.P;
        slice_ok = (unsigned)p < (unsigned)g.P;
    }
    if (!slice_ok) b = p = 0;
    const int tile = (int)blockIdx.x;
    const int ti = g.tiles_j == 1 ? tile : (int)__umulhi((unsigned)tile, g.tiles_j_magic);
    const int tj = tile - ti * g.tiles_j;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int j = tj * kTileJ + (warp & 1) * 8 + (lane & 7);
    const int i0 = ti * (2 * kTileI) + (warp >> 1) * 4 + (lane >> 3);
    const bool col_ok = slice_ok && j < g.Nh;
    const R* rm = pose_rot<DIM>(g, rot, b, p);
    // column terms, formed once for both pixels
    const R kc = (R)j;
    const R kc2 = mul_rn(kc, kc);
    const R sc = (sizeof(R) == 4 && g.os_is_float) ? mul_rn(kc, (R)g.os_f) : (R)((double)kc * g.os);
    R m_c[3], m_r[3];
    if (DIM == 3) {
        m_c[0] = mul_rn(__ldg(rm + 0), sc); m_r[0] = __ldg(rm + 1);
        m_c[1] = mul_rn(__ldg(rm + 3), sc); m_r[1] = __ldg(rm + 4);
        m_c[2] = mul_rn(__ldg(rm + 6), sc); m_r[2] = __ldg(rm + 7);
    } else {
        m_c[0] = mul_rn(__ldg(rm + 0), sc); m_r[0] = __ldg(rm + 1);
        m_c[1] = mul_rn(__ldg(rm + 2), sc); m_r[1] = __ldg(rm + 3);
        m_c[2] = 0.f; m_r[2] = 0.f;
    }
    R s0 = 0.f, kc_s1 = 0.f;
    if (g.has_shift) {
        const R* s = pose_shift(g, shifts, b, p);
        s0 = __ldg(s);
        kc_s1 = mul_rn(kc, __ldg(s + 1));
    }
    const C2<R>* vol = rec + (size_t)b * g.vol_elems;
    const size_t slice_base = (size_t)(b * g.P + p) * (size_t)g.slice_pixels;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int i = i0 + h * kTileI;
        const bool in_image = col_ok && i < g.N;
        PixelT<R> px;
        px.c = px.r = px.d = 0.f;
        px.kr = (R)((i <= g.N / 2) ? i : i - g.N);
        px.kc = kc;
        const R rad = add_rn(mul_rn(px.kr, px.kr), kc2);
        const bool valid = in_image && !(rad > cutoff_sq_of(g, rad));
        if (valid) {
            px.sc = sc;
            px.sr = (sizeof(R) == 4 && g.os_is_float) ? mul_rn(px.kr, (R)g.os_f) : (R)((double)px.kr * g.os);
            px.c = add_rn(m_c[0], mul_rn(m_r[0], px.sr));
            px.r = add_rn(m_c[1], mul_rn(m_r[1], px.sr));
            if (DIM == 3) px.d = add_rn(m_c[2], mul_rn(m_r[2], px.sr));
        }
        C2<R> v, gc, gr, gd;
        interpolate_any<DIM, false, false>(g, vol, px, valid, v, gc, gr, gd);      // all 32 lanes take part
        if (!in_image) continue;
        if (valid && g.has_shift) {
            const R dot = add_rn(mul_rn(px.kr, s0), kc_s1);
            const R ph = (R)((double)dot * g.phase_scale);
            R sn, cs;
            phase_sincos(ph, &sn, &cs);
            v = cmul(v, make2<R>(cs, sn));
        }
        __stcs(out + (slice_base + (size_t)(i * g.Nh + j)), v);
    }
}

// Pose-gradient terms shared by the two backward kernels.
//   rotation:  dL/dR[a][m] += s_m * Re(u * conj(grad_a)),  a: (c, r, d) rows, s = (sc, sr, 0)
//   shift:     dL/ds[n]    += q_n * (u.y * val.x - u.x * val.y),  q = -2*pi*k_n/N
template <int DIM, bool NEED_ROT, bool NEED_SHIFT, typename R>
__device__ __forceinline__ void pose_grad_terms(const SliceGeom& g, const PixelT<R>& px, C2<R> u_rot,
                                                C2<R> u_shift, C2<R> val_shift, C2<R> g_c,
                                                C2<R> g_r, C2<R> g_d,
                                                R (&acc)[2 * DIM + 2]) {
    if (NEED_ROT) {
        const R dc = u_rot.x * g_c.x + u_rot.y * g_c.y;
        const R dr = u_rot.x * g_r.x + u_rot.y * g_r.y;
        acc[0] += dc * px.sc;
        acc[1] += dc * px.sr;
        acc[2] += dr * px.sc;
        acc[3] += dr * px.sr;
        if (DIM == 3) {
            const R dd = u_rot.x * g_d.x + u_rot.y * g_d.y;
            acc[4] += dd * px.sc;
            acc[5] += dd * px.sr;
        }
    }
    if (NEED_SHIFT) {
        const R cross = u_shift.y * val_shift.x - u_shift.x * val_shift.y;
        acc[2 * DIM + 0] += (R)(g.shift_scale * (double)px.kr) * cross;
        acc[2 * DIM + 1] += (R)(g.shift_scale * (double)px.kc) * cross;
    }
}

template <int DIM, typename R>
__device__ __forceinline__ void pose_grad_flush(const SliceGeom& g, R (&acc)[2 * DIM + 2],
                                                R* grad_rot, R* grad_shift, int b, int p) {
    R* dst[2 * DIM + 2];
    R* gr = grad_rot ? grad_rot + (size_t)b * g.rot_stride_b + (size_t)p * (DIM * DIM) : nullptr;
    R* gs = grad_shift ? grad_shift + (size_t)b * g.shift_stride_b + (size_t)p * 2 : nullptr;
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
template <int DIM, bool CUBIC, bool NEED_ROT, bool NEED_SHIFT, typename R>
__global__ void __launch_bounds__(kBlockThreads, (DIM == 3 && CUBIC && NEED_ROT && sizeof(R) == 4) ? PB_MIN_BLOCKS : 1)
project_back_kernel(const C2<R>* __restrict__ grad_proj, const C2<R>* __restrict__ rec,
                    const R* __restrict__ rot, const R* __restrict__ shifts,
                    C2<R>* __restrict__ grad_rec, R* __restrict__ grad_rot,
                    R* __restrict__ grad_shift, const SliceGeom g) {
    const BlockWork w = block_work(g);
    R acc[2 * DIM + 2];
#pragma unroll
    for (int q = 0; q < 2 * DIM + 2; ++q) acc[q] = 0.f;
    PixelT<R> px;
    px.c = px.r = px.d = px.sc = px.sr = px.kr = px.kc = 0.f;
    const bool active = w.in_image &&
                        pixel_setup<DIM>(g, pose_rot<DIM>(g, rot, w.b, w.p), w.i, w.j, px) &&
                        !(w.j == 0 && w.i >= g.N / 2);
    C2<R> u = make2<R>(0.f, 0.f);
    if (active) {
        u = __ldcs(grad_proj + w.pix);
        if (g.has_shift) {
            const R* s = pose_shift(g, shifts, w.b, w.p);
            u = cmul_conj(u, phase_ramp(g, px, __ldg(s), __ldg(s + 1)));
        }
    }
    if (NEED_ROT || NEED_SHIFT) {
        // Pose gradients first, so that nothing but the pixel's position and `u` stays live across
        // the scatter below.  The gather returns the four real scalars they are made of (see
        // gather_pose_dots); every lane of the warp takes part in it.
        R dots[4];
        gather_pose_dots<DIM, CUBIC, NEED_ROT>(g, rec + (size_t)w.b * g.vol_elems, px, active, u, dots);
        if (active) {
            // the pixel's frequencies are formed again from (i, j) rather than kept in registers
            // across the gather (the empty asm keeps the compiler from reusing the earlier values)
            int i2 = w.i, j2 = w.j;
            asm volatile("" : "+r"(i2), "+r"(j2));
            const R kr = (R)((i2 <= g.N / 2) ? i2 : i2 - g.N), kc = (R)j2;
            if (NEED_ROT) {
                const R sc = (R)((double)kc * g.os), sr = (R)((double)kr * g.os);
#pragma unroll
                for (int a = 0; a < DIM; ++a) {
                    acc[2 * a + 0] = dots[a] * sc;
                    acc[2 * a + 1] = dots[a] * sr;
                }
            }
            if (NEED_SHIFT) {
                acc[2 * DIM + 0] = (R)(g.shift_scale * (double)kr) * dots[3];
                acc[2 * DIM + 1] = (R)(g.shift_scale * (double)kc) * dots[3];
            }
        }
        pose_grad_flush<DIM>(g, acc, grad_rot, grad_shift, w.b, w.p);
    }
    // cooperative scatter: every lane of the warp takes part
    scatter_coop<DIM, CUBIC, false, false, false>(g, grad_rec + (size_t)w.b * g.vol_elems, nullptr, nullptr,
                                                  px, active, u, 0.f);
}

// Backward of project_forw_saving_kernel: pose gradients from the saved derivatives and output
// (Re(grad * conj(derivative)) for the rotation, Im(grad * conj(output)) for the shift: the shift
// phase cancels in both), then the same scatter of the gradient into the volume (NEED_REC).
template <int DIM, bool CUBIC, bool NEED_ROT, bool NEED_SHIFT, bool NEED_REC>
__global__ void __launch_bounds__(kBlockThreads)
project_back_saved_kernel(const float2* __restrict__ grad_proj, const float2* __restrict__ out,
                          const float2* __restrict__ derivs, const float* __restrict__ rot,
                          const float* __restrict__ shifts, float2* __restrict__ grad_rec,
                          float* __restrict__ grad_rot, float* __restrict__ grad_shift, const SliceGeom g) {
    const BlockWork w = block_work(g);
    float acc[2 * DIM + 2];
#pragma unroll
    for (int q = 0; q < 2 * DIM + 2; ++q) acc[q] = 0.f;
    Pixel px;
    px.c = px.r = px.d = px.sc = px.sr = px.kr = px.kc = 0.f;
    const bool active = w.in_image &&
                        pixel_setup<DIM>(g, pose_rot<DIM>(g, rot, w.b, w.p), w.i, w.j, px) &&
                        !(w.j == 0 && w.i >= g.N / 2);
    float2 u = make_float2(0.f, 0.f);
    if (active) {
        u = __ldcs(grad_proj + w.pix);
        if (NEED_ROT) {
            const size_t plane = (size_t)g.BP * (size_t)g.slice_pixels;
#pragma unroll
            for (int a = 0; a < DIM; ++a) {
                const float2 d = __ldcs(derivs + (size_t)a * plane + w.pix);
                const float dot = u.x * d.x + u.y * d.y;
                acc[2 * a + 0] = dot * px.sc;
                acc[2 * a + 1] = dot * px.sr;
            }
        }
        if (NEED_SHIFT) {
            const float2 o = __ldcs(out + w.pix);
            const float cross = u.y * o.x - u.x * o.y;
            acc[2 * DIM + 0] = (float)(g.shift_scale * (double)px.kr) * cross;
            acc[2 * DIM + 1] = (float)(g.shift_scale * (double)px.kc) * cross;
        }
        if (NEED_REC && g.has_shift) {
            const float* s = pose_shift(g, shifts, w.b, w.p);
            u = cmul_conj(u, phase_ramp(g, px, __ldg(s), __ldg(s + 1)));
        }
    }
    if (NEED_ROT || NEED_SHIFT) pose_grad_flush<DIM>(g, acc, grad_rot, grad_shift, w.b, w.p);
    if (NEED_REC)
        scatter_coop<DIM, CUBIC, false, false, false>(g, grad_rec + (size_t)w.b * g.vol_elems, nullptr, nullptr,
                                                      px, active, u, 0.f);
}

// ---- back-projection --------------------------------------------------------------------
// reference semantics: csrc/cpu/3d/backprojection_2d_to_3d_kernels.cpp:177-291
// Slice value with the conjugate shift ramp applied, and its weight (shared by both kernels).
template <int DIM, bool WEIGHTS, typename R>
__device__ __forceinline__ bool backproject_pixel(const SliceGeom& g, const BlockWork& w,
                                                  const C2<R>* __restrict__ proj,
                                                  const R* __restrict__ weights,
                                                  const R* __restrict__ rot,
                                                  const R* __restrict__ shifts, PixelT<R>& px,
                                                  C2<R>& v, R& wv) {
    px.c = px.r = px.d = 0.f;
    v = make2<R>(0.f, 0.f);
    wv = 0.f;
    const bool active = w.in_image && !(w.j == 0 && w.i >= g.N / 2) &&
                        pixel_setup<DIM>(g, pose_rot<DIM>(g, rot, w.b, w.p), w.i, w.j, px);
    if (active) {
        v = __ldcs(proj + w.pix);
        if (g.has_shift) {
            const R* s = pose_shift(g, shifts, w.b, w.p);
            v = cmul_conj(v, phase_ramp(g, px, __ldg(s), __ldg(s + 1)));
        }
        if (WEIGHTS) wv = __ldcs(weights + w.pix);
    }
    return active;
}

template <int DIM, bool CUBIC, bool WEIGHTS, typename R>
__global__ void __launch_bounds__(kBlockThreads)
backproject_forw_kernel(const C2<R>* __restrict__ proj, const R* __restrict__ weights,
                        const R* __restrict__ rot, const R* __restrict__ shifts,
                        C2<R>* __restrict__ data_rec, R* __restrict__ weight_rec,
                        const SliceGeom g) {
    const BlockWork w = block_work(g);
    PixelT<R> px;
    C2<R> v;
    R wv;
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
    // A reconstruction of less than ~2 MB takes reductions at half the rate of a larger one (they pile
    // up on too few sectors), so the slices of a call are spread over g.replicas copies of it, which
    // the fold adds up.
    const size_t copy = (size_t)(w.p & (g.replicas - 1)) * (size_t)g.replica_stride;
    scatter_coop<DIM, CUBIC, true, true, true>(g, nullptr, nullptr, accum + copy + (size_t)w.b * g.vol_elems,
                                               px, active, v, wv);
}

// data[k] (+)= sum over copies of accum[k].xy, weight[k] (+)= sum over copies of accum[k].z
__global__ void __launch_bounds__(256)
fold_interleaved_kernel(const float4* __restrict__ accum, float2* __restrict__ data,
                        float* __restrict__ weight, size_t n, int accumulate, int replicas = 1,
                        size_t replica_stride = 0) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t k = (size_t)blockIdx.x * blockDim.x + threadIdx.x; k < n; k += stride) {
        float4 a = __ldcs(accum + k);
        for (int r = 1; r < replicas; ++r) {
            const float4 c = __ldcs(accum + (size_t)r * replica_stride + k);
            a.x += c.x;
            a.y += c.y;
            a.z += c.z;
        }
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

// out[k] = accum[k].xy / max(accum[k].z, eps): the weighted-average reconstruction straight from
// the interleaved accumulator (the fold and the division by the weights in one pass).
__global__ void __launch_bounds__(256)
fold_normalized_kernel(const float4* __restrict__ accum, float2* __restrict__ out, size_t n, float eps) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t k = (size_t)blockIdx.x * blockDim.x + threadIdx.x; k < n; k += stride) {
        const float4 a = __ldcs(accum + k);
        const float inv = 1.0f / fmaxf(a.z, eps);
        out[k] = make_float2(a.x * inv, a.y * inv);
    }
}

// ---- slab-ordered back-projection (3D, volumes larger than L2) ---------------------------
// When the accumulation volumes do not fit the 126 MB L2, reductions of the plain kernel miss
// it: consecutive slices have unrelated orientations, so a voxel is revisited only after
// gigabytes of other reductions, and every tap becomes a DRAM read-modify-write of a sector.
// This kernel reorders the work instead of the data: the volume is cut into slabs of
// `slab_planes` consecutive z planes (signed plane coordinates [z_lo, z_hi)) small enough to
// stay in L2, blockIdx.y walks the slabs (slowest grid index, so blocks of one slab run
// together) and, for its slab, each block visits only the pixels of its slice whose taps can
// land there.  Those pixels form, in every row of the slice, at most two runs of columns
// (d and c are linear in the column j; one run for direct taps, one for Friedel-mirrored
// taps, which land at -d and exist where c < 0); the runs are computed from linear estimates
// with a small slack, candidates pass a one-FMA prefilter, and each tap is then tested
// exactly (scatter_coop<SLAB>), so every tap is written by exactly one slab pass.  A pass writes
// only into the planes of its own slab: the Friedel duplicate of a tap on the c == 0 plane,
// which lands in the mirrored plane, is issued by the pass that owns THAT plane (pixels with a
// tap on column 0 are therefore candidates of the mirrored run as well).  So the planes of a
// slab are final as soon as its pass has run for every slice, which lets a caller fold and
// reduce a finished slab while later slabs are still being scattered (`slab_first` +
// gridDim.y select the slabs of a launch).
// One block = one slice x one slab; its 8 warps take the rows round-robin and each prepares 32
// of its rows at a time, one per lane.
// Restrict the column run [ja, jb] to the columns where a*j + b lies in [lo, hi]; inv_a = 1 / a
// (a is the same for every row of a slice, so the caller divides once per block).
__device__ __forceinline__ void clip_run(float a, float inv_a, float b, float lo, float hi, float& ja, float& jb) {
    if (fabsf(a) < 1e-6f) {
        if (b < lo || b > hi) jb = ja - 1.f;        // empty
        return;
    }
    const float x0 = (lo - b) * inv_a, x1 = (hi - b) * inv_a;
    ja = fmaxf(ja, fminf(x0, x1));
    jb = fminf(jb, fmaxf(x0, x1));
}

// INTERLEAVED: reductions go to a 16-byte-per-voxel (re, im, w, 0) accumulator `accum` (one v4
// reduction per tap) instead of data_rec / weight_rec.
template <bool CUBIC, bool WEIGHTS, bool INTERLEAVED = false>
__global__ void __launch_bounds__(kBlockThreads)
backproject_slab_kernel(const float2* __restrict__ proj, const float* __restrict__ weights,
                        const float* __restrict__ rot, const float* __restrict__ shifts,
                        float2* __restrict__ data_rec, float* __restrict__ weight_rec,
                        float4* __restrict__ accum, const SliceGeom g, int slab_planes, int slab_first) {
    constexpr int T = CUBIC ? 4 : 2;
    constexpr unsigned kFull = 0xffffffffu;
    constexpr float kEps = 0.05f;                    // slack of the linear estimates below
    const int bp = blockIdx.x;
    const int b = bp / g.P, p = bp - b * g.P;
    const int z_lo = -g.half + 1 + ((int)blockIdx.y + slab_first) * slab_planes;
    const int z_hi = min(z_lo + slab_planes, g.half + 1);
    const float* rm = pose_rot<3>(g, rot, b, p);
    // linear estimates of the sample position along a row: d ~ ad*j + bd*kr, c ~ ac*j + bc*kr
    const float osf = (float)g.os;
    const float ac = osf * __ldg(rm + 0), bc = osf * __ldg(rm + 1);
    const float ad = osf * __ldg(rm + 6), bd = osf * __ldg(rm + 7);
    const float inv_ac = 1.f / (fabsf(ac) < 1e-6f ? 1.f : ac), inv_ad = 1.f / (fabsf(ad) < 1e-6f ? 1.f : ad);
    // taps of a pixel use planes floor(d)-T/2+1 .. floor(d)+T/2 (mirrored taps their negatives)
    // and columns floor(c)-T/2+1 .. floor(c)+T/2; direct taps need a column >= 0, mirrored taps a
    // column < 0, and the duplicate of a column-0 tap (which lands in the mirrored plane) a column == 0
    const float band_lo = (float)z_lo - (float)(T / 2) - kEps;
    const float band_hi = (float)z_hi + (float)(T / 2 - 1) + kEps;
    const float c_direct_min = -(float)(T / 2) - kEps;
    const float c_mirror_max = (float)(T / 2) + kEps;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float2* data_b = INTERLEAVED ? nullptr : data_rec + (size_t)b * g.vol_elems;
    float* wrec_b = (WEIGHTS && !INTERLEAVED) ? weight_rec + (size_t)b * g.vol_elems : nullptr;
    float4* accum_b = INTERLEAVED ? accum + (size_t)b * g.vol_elems : nullptr;
    const float cut = sqrtf(g.cutoff_sq);
    // rows are dealt to the warps round-robin (row = n * 8 + warp), so that whichever rows a
    // slab's strip crosses, all warps of the block share them
    const int rows_per_warp = (g.N + kWarps - 1) / kWarps;

    for (int n0 = 0; n0 < rows_per_warp; n0 += 32) {
        // each lane prepares one row: its direct and mirrored column runs (empty: a > b)
        int run_a[2] = {1, 1}, run_b[2] = {0, 0};
        const int irow = (n0 + lane) * kWarps + warp;
        if (irow < g.N) {
            const float kr = (float)((irow <= g.N / 2) ? irow : irow - g.N);
            const float room = g.cutoff_sq - kr * kr;
            if (room >= 0.f) {
                const float jmax = fminf((float)(g.Nh - 1), fminf(sqrtf(room), cut) + 1.f);
                const float d0 = bd * kr, c0 = bc * kr;
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    float ja = 0.f, jb = jmax;
                    if (t == 0) {
                        clip_run(ad, inv_ad, d0, band_lo, band_hi, ja, jb);
                        clip_run(ac, inv_ac, c0, c_direct_min, 3.0e38f, ja, jb);
                    } else {
                        clip_run(ad, inv_ad, d0, -band_hi, -band_lo, ja, jb);
                        clip_run(ac, inv_ac, c0, -3.0e38f, c_mirror_max, ja, jb);
                    }
                    if (jb >= ja) {
                        // the bands carry kEps of slack in plane units, i.e. at least kEps / 2 columns: far more than
                        // the rounding of these estimates (< 1e-2 columns), so floor / ceil need no extra column
                        run_a[t] = max(0, (int)floorf(ja));
                        run_b[t] = min((int)jmax, (int)ceilf(jb));
                    }
                }
                // overlapping or adjacent runs become one (pixels must be visited once per slab)
                if (run_a[0] <= run_b[0] && run_a[1] <= run_b[1] &&
                    run_a[0] <= run_b[1] + 1 && run_a[1] <= run_b[0] + 1) {
                    run_a[0] = min(run_a[0], run_a[1]);
                    run_b[0] = max(run_b[0], run_b[1]);
                    run_a[1] = 1;
                    run_b[1] = 0;
                }
            }
        }
        // Flatten the candidate columns of these 32 rows into one index space so that the warp
        // stays full however thin the strips are: lane l holds n_l candidates, an inclusive
        // scan gives every row its offset, and candidate k finds its row by binary search.
        const int len0 = max(0, run_b[0] - run_a[0] + 1), len1 = max(0, run_b[1] - run_a[1] + 1);
        int incl = len0 + len1;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(kFull, incl, o);
            if (lane >= o) incl += up;
        }
        const int total = __shfl_sync(kFull, incl, 31);
        // candidate k of this batch of rows -> its pixel (i, j), whether this pass has work for it,
        // and its sample position
        auto candidate = [&](int k, int& i, int& j, Pixel& px) -> bool {
            // smallest row whose inclusive count exceeds k
            int row = 0;
#pragma unroll
            for (int step = 16; step > 0; step >>= 1) {
                const int probe = __shfl_sync(kFull, incl, (row + step - 1) & 31);
                if (k >= probe) row += step;
            }
            row = min(row, 31);
            const int r_incl = __shfl_sync(kFull, incl, row);
            const int r_len0 = __shfl_sync(kFull, len0, row), r_len1 = __shfl_sync(kFull, len1, row);
            const int r_a0 = __shfl_sync(kFull, run_a[0], row), r_a1 = __shfl_sync(kFull, run_a[1], row);
            const int local = k - (r_incl - r_len0 - r_len1);
            j = local < r_len0 ? r_a0 + local : r_a1 + (local - r_len0);
            i = (n0 + row) * kWarps + warp;
            const float kr = (float)((i <= g.N / 2) ? i : i - g.N);
            // one-FMA prefilter with the linear estimates, then the exact test
            const float de = fmaf(ad, (float)j, bd * kr), ce = fmaf(ac, (float)j, bc * kr);
            bool active = k < total && !(j == 0 && i >= g.N / 2) &&
                          ((de >= band_lo && de <= band_hi && ce >= c_direct_min) ||
                           (-de >= band_lo && -de <= band_hi && ce <= c_mirror_max));
            px.c = px.r = px.d = 0.f;
            if (active) active = pixel_setup<3>(g, rm, i, j, px);
            if (active) {
                const int pd = (int)floorf(px.d) - (CUBIC ? 1 : 0);
                const int pc = (int)floorf(px.c) - (CUBIC ? 1 : 0);
                const bool direct = pc + T - 1 >= 0 && pd < z_hi && pd + T > z_lo;
                const bool mirror = pc <= 0 && -(pd + T - 1) < z_hi && -pd >= z_lo;
                active = direct || mirror;
            }
            return active;
        };
        auto load_pixel = [&](bool active, int i, int j, float2& v, float& wv) {
            v = make_float2(0.f, 0.f);
            wv = 0.f;
            if (active) {
                const size_t pix = ((size_t)bp * (size_t)g.N + (size_t)i) * (size_t)g.Nh + (size_t)j;
                v = __ldcs(proj + pix);
                if (WEIGHTS) wv = __ldcs(weights + pix);
            }
        };
        auto scatter_pixel = [&](bool active, const Pixel& px, float2 v, float wv) {
            if (active && g.has_shift) {
                const float* s = pose_shift(g, shifts, b, p);
                v = cmul_conj(v, phase_ramp(g, px, __ldg(s), __ldg(s + 1)));
            }
            scatter_coop<3, CUBIC, WEIGHTS, true, INTERLEAVED, true>(g, data_b, wrec_b, accum_b, px, active, v, wv, z_lo, z_hi);
        };
        for (int k0 = 0; k0 < total; k0 += 32) {                                  // warp-uniform trip count
            int i, j;
            Pixel px;
            const bool active = candidate(k0 + lane, i, j, px);
            if (!__any_sync(kFull, active)) continue;
            float2 v;
            float wv;
            load_pixel(active, i, j, v, wv);
            scatter_pixel(active, px, v, wv);
        }
    }
}

// ---- backward of back-projection --------------------------------------------------------
// reference semantics: csrc/cpu/3d/backprojection_2d_to_3d_kernels.cpp:417-583
template <int DIM, bool CUBIC, bool NEED_ROT, bool NEED_SHIFT, typename R>
__global__ void __launch_bounds__(kBlockThreads)
backproject_back_kernel(const C2<R>* __restrict__ grad_data_rec,
                        const R* __restrict__ grad_weight_rec,
                        const C2<R>* __restrict__ proj, const R* __restrict__ rot,
                        const R* __restrict__ shifts, C2<R>* __restrict__ grad_proj,
                        R* __restrict__ grad_weights, R* __restrict__ grad_rot,
                        R* __restrict__ grad_shift, const SliceGeom g) {
    const BlockWork w = block_work(g);
    R acc[2 * DIM + 2];
#pragma unroll
    for (int q = 0; q < 2 * DIM + 2; ++q) acc[q] = 0.f;
    PixelT<R> px;
    px.c = px.r = px.d = px.sc = px.sr = px.kr = px.kc = 0.f;
    const bool active = w.in_image &&
                        pixel_setup<DIM>(g, pose_rot<DIM>(g, rot, w.b, w.p), w.i, w.j, px) &&
                        !(w.j == 0 && w.i >= g.N / 2);
    const bool write_w = grad_weight_rec != nullptr && grad_weights != nullptr;
    // the slice's own value with the conjugate shift ramp (what was back-projected): the pose
    // gradients are its dot products with the derivatives of the gathered gradient volume
    C2<R> ph = make2<R>(1.f, 0.f), pv = make2<R>(0.f, 0.f);
    if (active) {
        if (g.has_shift) {
            const R* s = pose_shift(g, shifts, w.b, w.p);
            ph = phase_ramp(g, px, __ldg(s), __ldg(s + 1));
        }
        if (NEED_ROT || NEED_SHIFT) {
            pv = __ldcs(proj + w.pix);
            if (g.has_shift) pv = cmul_conj(pv, ph);
        }
    }
    C2<R> raw;
    R dots[4];
    // cooperative gather: every lane of the warp takes part
    gather_pose_dots<DIM, CUBIC, NEED_ROT, true>(g, grad_data_rec + (size_t)w.b * g.vol_elems, px, active, pv, dots, &raw);
    if (active) {
        __stcs(grad_proj + w.pix, g.has_shift ? cmul(raw, ph) : raw);
        if (write_w)
            __stcs(grad_weights + w.pix,
                   gather_weight_grad<DIM>(g, grad_weight_rec + (size_t)w.b * g.vol_elems, px));
        if (NEED_ROT) {
#pragma unroll
            for (int a = 0; a < DIM; ++a) {
                acc[2 * a + 0] = dots[a] * px.sc;
                acc[2 * a + 1] = dots[a] * px.sr;
            }
        }
        if (NEED_SHIFT) {
            acc[2 * DIM + 0] = (R)(g.shift_scale * (double)px.kr) * dots[3];
            acc[2 * DIM + 1] = (R)(g.shift_scale * (double)px.kc) * dots[3];
        }
    } else if (w.in_image) {
        __stcs(grad_proj + w.pix, make2<R>(0.f, 0.f));
        if (write_w) __stcs(grad_weights + w.pix, 0.f);
    }
    if (NEED_ROT || NEED_SHIFT) pose_grad_flush<DIM>(g, acc, grad_rot, grad_shift, w.b, w.p);
}

// ---- processing order of the slices of a 3D operator --------------------------------------
// Slices whose planes lie close together read (nearly) the same voxels.  When the volume is
// larger than L2, running them one after the other turns most of those reads into L2 hits,
// which random pose order does not.  The key is the slice normal (third column of the
// rotation matrix, flipped into the upper hemisphere: n and -n span the same plane), mapped
// to the unit disc by an equal-area projection and quantised to a 32 x 32 grid walked in
// Morton order.  One block per batch item counting-sorts its P poses by that key: a histogram
// in shared memory, an exclusive scan, then each pose takes the next free place of its bin.
// The order inside a bin depends on thread timing; results of the operators do not depend on
// the processing order at all.
constexpr int kOrderBits = 5;
constexpr int kOrderBins = 1 << (2 * kOrderBits);

template <typename R>
__device__ __forceinline__ int pose_order_key(const R* __restrict__ rm) {
    float nx = (float)__ldg(rm + 2), ny = (float)__ldg(rm + 5), nz = (float)__ldg(rm + 8);
    if (nz < 0.f) { nx = -nx; ny = -ny; nz = -nz; }
    const float s = rsqrtf(fmaxf(1.f + nz, 1e-6f));          // |(nx, ny)| * s <= 1 on the hemisphere
    const float q = (float)(1 << kOrderBits);
    // min/max also send a NaN to a valid cell
    const int x = (int)fminf(fmaxf((nx * s * 0.5f + 0.5f) * q, 0.f), q - 1.f);
    const int y = (int)fminf(fmaxf((ny * s * 0.5f + 0.5f) * q, 0.f), q - 1.f);
    int key = 0;
#pragma unroll
    for (int k = 0; k < kOrderBits; ++k) key |= ((x >> k) & 1) << (2 * k) | ((y >> k) & 1) << (2 * k + 1);
    return key;
}

template <typename R>
__global__ void __launch_bounds__(kOrderBins)
pose_order_kernel(const R* __restrict__ rot, long long rot_stride_b, int P, int* __restrict__ order) {
    __shared__ int bins[kOrderBins];
    __shared__ int warp_sum[kOrderBins / 32];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const R* rm = rot + (size_t)blockIdx.x * (size_t)rot_stride_b;
    const int base = (int)blockIdx.x * P;
    bins[t] = 0;
    __syncthreads();
    for (int p = t; p < P; p += kOrderBins) atomicAdd(&bins[pose_order_key(rm + (size_t)p * 9)], 1);
    __syncthreads();
    // exclusive scan of the 1024 counts: inside each warp, then over the 32 warp totals
    const int count = bins[t];
    int incl = count;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += up;
    }
    if (lane == 31) warp_sum[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        const int total = warp_sum[lane];
        int w = total;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, w, d);
            if (lane >= d) w += up;
        }
        warp_sum[lane] = w - total;
    }
    __syncthreads();
    bins[t] = warp_sum[warp] + incl - count;
    __syncthreads();
    for (int p = t; p < P; p += kOrderBins) {
        const int pos = atomicAdd(&bins[pose_order_key(rm + (size_t)p * 9)], 1);
        order[base + pos] = base + p;
    }
}

// ---- reduction-rate probe -------------------------------------------------------------------
// How many red.global.add the memory system retires per second for the access patterns of the
// scatter kernels, on a buffer the caller sizes (L2-resident: the ceiling of the scatters; far
// beyond L2: what they fall to when the volume does not fit).  Every lane issues `iters`
// reductions to pseudo-random places:
//   0  one random 16-byte slot per lane                      (red.v4)
//   1  lane pairs on two adjacent 16-byte slots              (red.v4; the linear scatter into an interleaved volume)
//   2  lane pairs on the two halves of one 32-byte sector    (red.v4)
//   3  four lanes on four adjacent 8-byte voxels             (red.v2; the cubic scatter into a complex volume)
//   4  one random 8-byte voxel per lane                      (red.v2)
//   5  lane pairs on two adjacent 8-byte voxels              (red.v2; the linear scatter into a complex volume)
__device__ __forceinline__ unsigned probe_hash(unsigned x) {
    x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
    return x;
}

template <int PATTERN>
__global__ void __launch_bounds__(256)
reduction_rate_kernel(float* __restrict__ buf, unsigned units, int iters) {
    // units: 16-byte slots (patterns 0-2) or 8-byte voxels (3-5) in the buffer
    const unsigned t = blockIdx.x * blockDim.x + threadIdx.x;
    for (int i = 0; i < iters; ++i) {
        if (PATTERN == 0) {
            const unsigned s = probe_hash(t * 977u + i * 7919u) % units;
            red_add_v4(reinterpret_cast<float4*>(buf) + s, 1.f, 1.f, 1.f, 0.f);
        } else if (PATTERN == 1) {
            const unsigned s = probe_hash((t >> 1) * 977u + i * 7919u) % (units - 1) + (t & 1);
            red_add_v4(reinterpret_cast<float4*>(buf) + s, 1.f, 1.f, 1.f, 0.f);
        } else if (PATTERN == 2) {
            const unsigned s = (probe_hash((t >> 1) * 977u + i * 7919u) % (units / 2)) * 2 + (t & 1);
            red_add_v4(reinterpret_cast<float4*>(buf) + s, 1.f, 1.f, 1.f, 0.f);
        } else if (PATTERN == 3) {
            const unsigned s = probe_hash((t >> 2) * 977u + i * 7919u) % (units - 3) + (t & 3);
            red_add_v2(reinterpret_cast<float2*>(buf) + s, 1.f, 1.f);
        } else if (PATTERN == 4) {
            const unsigned s = probe_hash(t * 977u + i * 7919u) % units;
            red_add_v2(reinterpret_cast<float2*>(buf) + s, 1.f, 1.f);
        } else {
            const unsigned s = probe_hash((t >> 1) * 977u + i * 7919u) % (units - 1) + (t & 1);
            red_add_v2(reinterpret_cast<float2*>(buf) + s, 1.f, 1.f);
        }
    }
}

// The memory traffic of the slab-ordered scatter, without its arithmetic: lane pairs add to adjacent
// 16-byte slots inside a window of `window` slots that moves through the target as the grid
// advances (block b works in window b * n_windows / gridDim.x, as the slab index is the slow grid
// axis there), and every lane streams 8 bytes per four reductions from `src` (the slices).  With a
// window that fits L2, a target far beyond it and ~16 reductions per slot of a window this has the
// kernel's proportions: 2 bytes per tap of target fill + write-back, 2 bytes per tap streamed.
// KEEP: the reductions carry the L2 evict-last hint that the slab-ordered kernel gives them.
template <bool KEEP>
__global__ void __launch_bounds__(256)
reduction_stream_kernel(float* __restrict__ buf, unsigned units, unsigned window,
                        const float2* __restrict__ src, unsigned src_units, int iters) {
    const unsigned t = blockIdx.x * blockDim.x + threadIdx.x;
    const unsigned n_windows = units / window;
    const unsigned base = (unsigned)(((unsigned long long)blockIdx.x * n_windows) / gridDim.x) * window;
    const unsigned per_block = (unsigned)(iters + 3) / 4;
    float2 v = make_float2(0.f, 0.f);
    for (int i = 0; i < iters; ++i) {
        if ((i & 3) == 0) {
            const unsigned long long k = ((unsigned long long)blockIdx.x * per_block + (unsigned)(i >> 2)) * 256u + threadIdx.x;
            v = __ldcs(src + (unsigned)(k % src_units));
        }
        const unsigned s = base + probe_hash((t >> 1) * 977u + i * 7919u) % (window - 1) + (t & 1);
        if (KEEP) red_add_v4_keep(reinterpret_cast<float4*>(buf) + s, 1.f, 1.f + v.x, 1.f + v.y, 0.f, l2_keep_policy());
        else red_add_v4(reinterpret_cast<float4*>(buf) + s, 1.f, 1.f + v.x, 1.f + v.y, 0.f);
    }
}

// ---- the steps either side of the operators: pad + fftshift, ifftshift + crop ----------------
// Real-space image / volume (box n) <-> zero-padded, origin-at-index-0 array (box m >= n, both
// even or n odd is fine; lo = (m - n) / 2) that cuFFT transforms.  One pass each instead of
// pad -> roll (two extra passes over the padded array).
//   pad:   out[i...] = in[s(i0), s(i1)(, s(i2))],  s(i) = (i + m/2) mod m - lo,  0 outside [0, n)
//   crop:  out[j...] = in[t(j0), t(j1)(, t(j2))],  t(j) = (j + lo + m/2) mod m
// The two are adjoint to each other, which is what autograd needs.
// Block = 64 x 4 threads: a thread produces 4 consecutive elements of one row (one 16-byte
// store when VEC: the output rows are then 16-byte aligned), a block 256 elements of 4 rows.
// Grid: x covers the innermost axis, y the middle axis, z = batch * (outer axis or 1).
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(double* p, const double (&v)[4]) {
    *reinterpret_cast<double2*>(p) = make_double2(v[0], v[1]);
    *reinterpret_cast<double2*>(p + 2) = make_double2(v[2], v[3]);
}

template <int DIMS, bool PAD, bool VEC, typename R>
__global__ void __launch_bounds__(256)
pad_shift_kernel(const R* __restrict__ in, R* __restrict__ out, int n, int m, int lo, int batch) {
    const int out_box = PAD ? m : n, in_box = PAD ? n : m;
    const int j0 = (int)(blockIdx.x * 64 + threadIdx.x) * 4;
    const int i1 = (int)(blockIdx.y * 4 + threadIdx.y);
    const int zi = (int)blockIdx.z;
    const int b = DIMS == 3 ? zi / out_box : zi;
    const int i0 = DIMS == 3 ? zi - b * out_box : 0;
    if (j0 >= out_box || i1 >= out_box || b >= batch) return;
    const int half = m / 2;
    auto src = [&](int i) {
        if (PAD) { int s = i + half; if (s >= m) s -= m; return s - lo; }
        int t = i + lo + half; if (t >= m) t -= m; return t;
    };
    const int s1 = src(i1), s0 = DIMS == 3 ? src(i0) : 0;
    const bool row_ok = !PAD || ((unsigned)s1 < (unsigned)n && (unsigned)s0 < (unsigned)n);
    const size_t in_row = ((size_t)((long long)b * (DIMS == 3 ? in_box : 1) + s0) * in_box + s1) * in_box;
    const size_t o = ((size_t)((long long)b * (DIMS == 3 ? out_box : 1) + i0) * out_box + i1) * out_box + j0;
    R v[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        v[q] = 0;
        const int s2 = src(j0 + q);
        if (row_ok && j0 + q < out_box && (!PAD || (unsigned)s2 < (unsigned)n))
            v[q] = PAD ? __ldg(in + in_row + s2) : __ldcs(in + in_row + s2);
    }
    if (VEC) {
        store4(out + o, v);
    } else {
#pragma unroll
        for (int q = 0; q < 4; ++q)
            if (j0 + q < out_box) out[o + q] = v[q];
    }
}

}  // namespace b200proj
