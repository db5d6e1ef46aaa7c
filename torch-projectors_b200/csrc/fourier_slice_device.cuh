// Device-side building blocks of the sm_100a Fourier-slice kernels: pixel -> sample
// geometry, separable interpolation weights, gather (clamping) and scatter (dropping)
// footprints in the rfft half-volume, phase ramps and block reductions.
//
// Numerical contract (reference: csrc/cpu in warpem/torch-projectors, the CPU backend is
// the parity target):
//  * sample coordinates reproduce the reference's fp32 rounding sequence exactly
//    (csrc/cpu/3d/projection_3d_to_2d_kernels.cpp:163-188): k*os is formed in double and
//    rounded once, the rotation is separately rounded fp32 multiplies and adds (no FMA),
//    so floor() and the fractional parts agree bit for bit with the CPU result;
//  * the phase of the shift ramp is float(double(float(kr*s0 + kc*s1)) * (-2*pi/N))
//    (csrc/cpu/common/projection_utils.h:82-94); fp32: reduced to about [-pi, pi] by a
//    two-constant Cody-Waite step in fp32 and evaluated with the hardware sin/cos
//    (see phase_sincos); fp64: the library sincos;
//  * tap sums are re-associated (separable form); that moves results by ~1e-7 relative.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace b200proj {

constexpr int kTileJ = 16;            // block tile: 16 columns x 16 rows of one slice
constexpr int kTileI = 16;
constexpr int kBlockThreads = kTileJ * kTileI;
constexpr int kWarps = kBlockThreads / 32;

// ---- real-type helpers -------------------------------------------------------------------
// The device code is generic over R = float (complex64 tensors, the fast path) and R = double
// (complex128 / float64, for callers that verify gradients in double precision, as the
// reference's own gradcheck tests do).  R is the last template parameter of every function
// and is deduced from the arguments.
template <typename R> struct Vec2;
template <> struct Vec2<float> { using type = float2; };
template <> struct Vec2<double> { using type = double2; };
template <typename R> using C2 = typename Vec2<R>::type;
// a parameter type that takes no part in the deduction of R (R comes from the pixel argument)
template <typename R> struct Identity { using type = R; };
template <typename R> using NoDeduce = typename Identity<R>::type;

template <typename R> __device__ __forceinline__ C2<R> make2(R a, R b);
template <> __device__ __forceinline__ float2 make2<float>(float a, float b) { return make_float2(a, b); }
template <> __device__ __forceinline__ double2 make2<double>(double a, double b) { return make_double2(a, b); }

__device__ __forceinline__ float rfloor(float x) { return floorf(x); }
__device__ __forceinline__ double rfloor(double x) { return floor(x); }
__device__ __forceinline__ float rabs(float x) { return fabsf(x); }
__device__ __forceinline__ double rabs(double x) { return fabs(x); }
__device__ __forceinline__ float rfma(float a, float b, float c) { return fmaf(a, b, c); }
__device__ __forceinline__ double rfma(double a, double b, double c) { return fma(a, b, c); }
// separately rounded multiply / add (never contracted into an FMA)
__device__ __forceinline__ float mul_rn(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ double mul_rn(double a, double b) { return __dmul_rn(a, b); }
__device__ __forceinline__ float add_rn(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ double add_rn(double a, double b) { return __dadd_rn(a, b); }

// Kernel parameters shared by the eight operators (passed by value).
struct SliceGeom {
    int N, Nh;              // projection box and stored width N/2+1
    int R, Rh, half;        // volume box, stored width R/2+1, R/2
    int P;                  // poses per batch item
    int BP;                 // B * P, slices of the call
    int decode;             // how (blockIdx.y, blockIdx.z) name a slice: 0 = one batch item, p = y + 32768*z;
                            // 1 = b = z, p = y; 2 = b*P + p = y + 32768*z (needs a division)
    int slice_pixels;       // N * Nh
    int os_is_float;        // the oversampling factor is exactly representable in float
    float os_f;
    int sparse_samples;     // oversampling >= 1.5
    unsigned tiles_j_magic; // ceil(2^32 / tiles_j): tile / tiles_j == __umulhi(tile, magic) for tile < 2^16
    int tiles_j, tiles_i;   // block tiles per slice
    int rot_stride_b;       // elements between batch items of rot (0 = shared)
    int shift_stride_b;     // elements between batch items of shifts (0 = shared)
    int has_shift;
    float cutoff_sq;        // (float(cutoff))^2, the fp32 path compares in float as the reference does
    double cutoff_sq_d;     // cutoff^2 for the fp64 path
    double os;              // oversampling factor
    double phase_scale;     // -2*pi / float(N)
    double shift_scale;     // -2*pi / N   (d phase / d shift per unit frequency)
    long long vol_elems;    // voxels per batch item
    const int* order;       // optional processing order: block k handles slice order[k] (a permutation of
                            // [0, BP)); nullptr = natural order.  Changes which blocks run together, not results.
    int replicas;           // interleaved workspace of a small reconstruction: number of copies (a power of two) the
    long long replica_stride;   // slices are spread over, and the voxels between copies; 1 / 0 = a single copy
    const int* pack_index;  // packed output of the forward projection: position of pixel i*Nh + j among the
    int pack_count;         // pack_count pixels inside the cutoff (-1 outside); nullptr = dense [N, Nh] slices
};

template <typename R>
struct PixelT {
    R kr, kc;           // projection frequencies (row, column)
    R sc, sr;           // oversampled sample coordinates before rotation
    R c, r, d;          // rotated sample position in the volume (x, y, z)
};
using Pixel = PixelT<float>;

// Lane -> pixel inside the block tile.  A warp covers 8 columns x 4 rows so that its
// samples form a compact patch of the slice plane (cache locality of the taps) while each
// row segment is 64 contiguous bytes of the output.
__device__ __forceinline__ void tile_pixel(const SliceGeom& g, int tile, int& i, int& j) {
    // tile / tiles_j without a division (a single tile column has no 32-bit magic number)
    const int ti = g.tiles_j == 1 ? tile : (int)__umulhi((unsigned)tile, g.tiles_j_magic);
    const int tj = tile - ti * g.tiles_j;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    j = tj * kTileJ + (warp & 1) * 8 + (lane & 7);
    i = ti * kTileI + (warp >> 1) * 4 + (lane >> 3);
}

__device__ __forceinline__ float cutoff_sq_of(const SliceGeom& g, float) { return g.cutoff_sq; }
__device__ __forceinline__ double cutoff_sq_of(const SliceGeom& g, double) { return g.cutoff_sq_d; }

// Frequencies, cutoff test and rotated sample position of output pixel (i, j).
// Returns false when the pixel lies outside the cutoff radius.
template <int DIM, typename R>
__device__ __forceinline__ bool pixel_setup(const SliceGeom& g, const R* __restrict__ rm,
                                            int i, int j, PixelT<R>& px) {
    px.kr = (R)((i <= g.N / 2) ? i : i - g.N);
    px.kc = (R)j;
    const R rad = add_rn(mul_rn(px.kr, px.kr), mul_rn(px.kc, px.kc));
    if (rad > cutoff_sq_of(g, rad)) return false;
    if (sizeof(R) == 4 && g.os_is_float) {
        // the exact product of two floats rounds to the same float from double or in one fp32 multiply
        px.sc = mul_rn(px.kc, (R)g.os_f);
        px.sr = mul_rn(px.kr, (R)g.os_f);
    } else {
        px.sc = (R)((double)px.kc * g.os);
        px.sr = (R)((double)px.kr * g.os);
    }
    if (DIM == 3) {
        px.c = add_rn(mul_rn(__ldg(rm + 0), px.sc), mul_rn(__ldg(rm + 1), px.sr));
        px.r = add_rn(mul_rn(__ldg(rm + 3), px.sc), mul_rn(__ldg(rm + 4), px.sr));
        px.d = add_rn(mul_rn(__ldg(rm + 6), px.sc), mul_rn(__ldg(rm + 7), px.sr));
    } else {
        px.c = add_rn(mul_rn(__ldg(rm + 0), px.sc), mul_rn(__ldg(rm + 1), px.sr));
        px.r = add_rn(mul_rn(__ldg(rm + 2), px.sc), mul_rn(__ldg(rm + 3), px.sr));
        px.d = 0.f;
    }
    return true;
}

// sin and cos of a phase of tens of radians.  fp32: the phase (already rounded to float as the
// reference rounds it) is reduced to about [-pi, pi] with a two-constant Cody-Waite step in
// fp32 (2*pi = 6.28125 + 1.9353072e-3: the first product is exact for |k| < 2^16, so the
// reduced argument is good to ~1e-7), then evaluated with the hardware approximations, whose
// absolute error there (< 5e-7) is below the fp32 noise of the interpolated value it
// multiplies; this replaces ~40 instructions of sincosf's full-range path by 6.  fp64: the
// accurate library routine.
__device__ __forceinline__ void phase_sincos(float ph, float* sn, float* cs) {
    const float k = rintf(ph * 0.15915494309189535f);               // 1 / (2*pi)
    float r = fmaf(k, -6.28125f, ph);
    r = fmaf(k, -1.9353071795864769e-3f, r);
    *sn = __sinf(r);
    *cs = __cosf(r);
}
__device__ __forceinline__ void phase_sincos(double ph, double* sn, double* cs) { sincos(ph, sn, cs); }

// exp(-2*pi*i*(kr*s0 + kc*s1)/N) as (cos, sin).
template <typename R>
__device__ __forceinline__ C2<R> phase_ramp(const SliceGeom& g, const PixelT<R>& px, R s0, R s1) {
    const R dot = add_rn(mul_rn(px.kr, s0), mul_rn(px.kc, s1));
    const R ph = (R)((double)dot * g.phase_scale);
    R sn, cs;
    phase_sincos(ph, &sn, &cs);
    return make2<R>(cs, sn);
}

template <typename V>
__device__ __forceinline__ V cmul(V a, V b) {
    V o;
    o.x = a.x * b.x - a.y * b.y;
    o.y = a.x * b.y + a.y * b.x;
    return o;
}
template <typename V>
__device__ __forceinline__ V cmul_conj(V a, V b) {   // a * conj(b)
    V o;
    o.x = a.x * b.x + a.y * b.y;
    o.y = a.y * b.x - a.x * b.y;
    return o;
}

// Catmull-Rom (a = -0.5) weights of the four taps floor-1 .. floor+2 for a fractional position
// f in [0, 1), and their derivatives with respect to f.  These are the polynomials
// w(f - t), t = -1..2, of the reference's piecewise kernel
// (csrc/cpu/common/cubic_kernels.h:25-66) written out per tap, so that no branch on |s| is needed.
template <typename R>
__device__ __forceinline__ void cubic_weights(R f, R (&w)[4]) {
    w[0] = ((-0.5f * f + 1.0f) * f - 0.5f) * f;
    w[1] = (1.5f * f - 2.5f) * f * f + 1.0f;
    w[2] = ((-1.5f * f + 2.0f) * f + 0.5f) * f;
    w[3] = (0.5f * f - 0.5f) * f * f;
}
template <typename R>
__device__ __forceinline__ void cubic_dweights(R f, R (&dw)[4]) {
    dw[0] = (-1.5f * f + 2.0f) * f - 0.5f;
    dw[1] = (4.5f * f - 5.0f) * f;
    dw[2] = (-4.5f * f + 4.0f) * f + 0.5f;
    dw[3] = (1.5f * f - 1.0f) * f;
}

// One of those weights / derivatives (tap K = 0..3), for code that wants them one at a time
// instead of holding all four in registers.
template <int K, typename R>
__device__ __forceinline__ R cubic_weight_k(R f) {
    if (K == 0) return ((-0.5f * f + 1.0f) * f - 0.5f) * f;
    if (K == 1) return (1.5f * f - 2.5f) * f * f + 1.0f;
    if (K == 2) return ((-1.5f * f + 2.0f) * f + 0.5f) * f;
    return (0.5f * f - 0.5f) * f * f;
}
template <int K, typename R>
__device__ __forceinline__ R cubic_dweight_k(R f) {
    if (K == 0) return (-1.5f * f + 2.0f) * f - 0.5f;
    if (K == 1) return (4.5f * f - 5.0f) * f;
    if (K == 2) return (-4.5f * f + 4.0f) * f + 0.5f;
    return (1.5f * f - 1.0f) * f;
}

// Per-axis interpolation weights: T = 2 (linear: taps at floor, floor+1) or
// T = 4 (cubic: taps at floor-1 .. floor+2).  base = index of the first tap.
template <typename R, int T>
struct AxisWeights {
    int base;
    R w[T];
    R dw[T];
};

template <int T, bool WITH_DERIV, typename R>
__device__ __forceinline__ void axis_weights(R x, AxisWeights<R, T>& a) {
    const R fl = rfloor(x);
    const R f = x - fl;
    if constexpr (T == 2) {
        a.base = (int)fl;
        a.w[0] = 1.f - f;
        a.w[1] = f;
        if (WITH_DERIV) { a.dw[0] = -1.f; a.dw[1] = 1.f; }
    } else {
        a.base = (int)fl - 1;
        cubic_weights(f, a.w);
        if (WITH_DERIV) cubic_dweights(f, a.dw);
    }
}

// ---- gather addressing (values outside the stored half-volume replicate the edge) -------
// reference: csrc/cpu/common/fftw_sampling.h:96-137 and, for cubic, the pre-clamp of
// csrc/cpu/common/interpolation_kernels.h:331-342.

// Integer min / max usable from host code too (the index helpers below are also compiled for
// the host, where a unit test feeds them INT_MIN / INT_MAX).
__host__ __device__ __forceinline__ int imin(int a, int b) { return a < b ? a : b; }
__host__ __device__ __forceinline__ int imax(int a, int b) { return a > b ? a : b; }

// Column index of signed column c; `mirrored` tells whether the Friedel mate is read.
// The column is clamped to [-(Rh-1), Rh-1] BEFORE the mirror: for in-range and moderately
// out-of-range columns that equals "mirror, then clamp to Rh-1" (linear) and the cubic
// pre-clamp, and it keeps a saturated coordinate (INT_MIN from a sample position at or below
// -2^31, whose negation is INT_MIN again) from becoming a negative index.
template <bool CUBIC>
__host__ __device__ __forceinline__ int gather_col(const SliceGeom& g, int c, bool& mirrored) {
    c = imax(-(g.Rh - 1), imin(c, g.Rh - 1));
    mirrored = c < 0;
    return mirrored ? -c : c;
}

// Row / plane index of signed coordinate r, for a tap that is (not) mirrored.
template <bool CUBIC>
__host__ __device__ __forceinline__ int gather_line(const SliceGeom& g, int r, bool mirrored) {
    if (CUBIC) r = imax(-g.half + 1, imin(r, g.half));
    if (mirrored) r = -r;                          // INT_MIN stays INT_MIN, which the clamp below catches
    r = imin(g.half, imax(r, -g.half + 1));
    return r < 0 ? r + g.R : r;
}

// Two floats in one 64-bit register and the packed fused multiply-add on them (sm_100).
__device__ __forceinline__ unsigned long long pack2(float x, float y) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(x), "f"(y));
    return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& x, float& y) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(x), "=f"(y) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

// One-lane-per-pixel separable interpolation (used for linear interpolation, whose 2-tap rows
// are too short for lane groups to pay for their shuffles: the linear gathers are bound by
// instruction issue, not by the L1TEX data pipe).  Same value and derivative conventions as
// interpolate_coop.
template <int DIM, bool CUBIC, bool WITH_DERIV, typename R>
__device__ __forceinline__ void interpolate_lane(const SliceGeom& g, const C2<R>* __restrict__ vol,
                                                 const PixelT<R>& px, C2<R>& val, C2<R>& g_c,
                                                 C2<R>& g_r, C2<R>& g_d) {
    constexpr int T = CUBIC ? 4 : 2;
    constexpr int TD = (DIM == 3) ? T : 1;
    AxisWeights<R, T> ac, ar, ad;
    axis_weights<T, WITH_DERIV>(px.c, ac);
    axis_weights<T, WITH_DERIV>(px.r, ar);
    if (DIM == 3) axis_weights<T, WITH_DERIV>(px.d, ad);
    const int plane_stride = g.R * g.Rh;
    val = make2<R>(0.f, 0.f);
    g_c = g_r = g_d = val;
    const bool interior = ar.base >= -g.half + 1 && ar.base + T - 1 <= g.half - 1 &&
                          (DIM == 2 || (ad.base >= -g.half + 1 && ad.base + T - 1 <= g.half - 1));
    if constexpr (sizeof(R) == 4 && !WITH_DERIV) {
        // fp32, value only: packed two-wide fused multiply-adds for the complex sums (see coop_column_sums)
        unsigned long long w2[T], val2 = 0ull;
#pragma unroll
        for (int i = 0; i < T; ++i) w2[i] = pack2(ar.w[i], ar.w[i]);
#pragma unroll
        for (int j = 0; j < T; ++j) {
            bool m;
            const int col = gather_col<CUBIC>(g, ac.base + j, m);
            unsigned long long A2 = 0ull;
#pragma unroll
            for (int k = 0; k < TD; ++k) {
                int pl = 0;
                if (DIM == 3) {
                    if (interior) {
                        const int d = m ? -(ad.base + k) : ad.base + k;
                        pl = (d < 0 ? d + g.R : d) * plane_stride;
                    } else {
                        pl = gather_line<CUBIC>(g, ad.base + k, m) * plane_stride;
                    }
                }
                unsigned long long rs2 = 0ull;
#pragma unroll
                for (int i = 0; i < T; ++i) {
                    int rw;
                    if (interior) {
                        const int r = m ? -(ar.base + i) : ar.base + i;
                        rw = (r < 0 ? r + g.R : r) * g.Rh;
                    } else {
                        rw = gather_line<CUBIC>(g, ar.base + i, m) * g.Rh;
                    }
                    const float2 v = __ldg((const float2*)vol + (pl + rw + col));
                    rs2 = fma2(w2[i], pack2(v.x, v.y), rs2);
                }
                const float wd = (DIM == 3) ? (float)ad.w[k] : 1.f;
                A2 = fma2(pack2(wd, wd), rs2, A2);
            }
            const float wc = (float)ac.w[j];
            val2 = fma2(pack2(wc, m ? -wc : wc), A2, val2);
        }
        float vx, vy;
        unpack2(val2, vx, vy);
        val = make2<R>(vx, vy);
    } else {
#pragma unroll
    for (int j = 0; j < T; ++j) {
        bool m;
        const int col = gather_col<CUBIC>(g, ac.base + j, m);
        C2<R> A = make2<R>(0.f, 0.f), Bq = A, Dq = A;
#pragma unroll
        for (int k = 0; k < TD; ++k) {
            int pl = 0;
            if (DIM == 3) {
                if (interior) {
                    const int d = m ? -(ad.base + k) : ad.base + k;
                    pl = (d < 0 ? d + g.R : d) * plane_stride;
                } else {
                    pl = gather_line<CUBIC>(g, ad.base + k, m) * plane_stride;
                }
            }
            C2<R> rs = make2<R>(0.f, 0.f), rds = rs;
#pragma unroll
            for (int i = 0; i < T; ++i) {
                int rw;
                if (interior) {
                    const int r = m ? -(ar.base + i) : ar.base + i;
                    rw = (r < 0 ? r + g.R : r) * g.Rh;
                } else {
                    rw = gather_line<CUBIC>(g, ar.base + i, m) * g.Rh;
                }
                const C2<R> v = __ldg(vol + (pl + rw + col));
                rs.x = rfma(ar.w[i], v.x, rs.x);
                rs.y = rfma(ar.w[i], v.y, rs.y);
                if (WITH_DERIV) {
                    rds.x = rfma(ar.dw[i], v.x, rds.x);
                    rds.y = rfma(ar.dw[i], v.y, rds.y);
                }
            }
            const R wd = (DIM == 3) ? ad.w[k] : (R)1;
            A.x = rfma(wd, rs.x, A.x);
            A.y = rfma(wd, rs.y, A.y);
            if (WITH_DERIV) {
                Bq.x = rfma(wd, rds.x, Bq.x);
                Bq.y = rfma(wd, rds.y, Bq.y);
                if (DIM == 3) {
                    Dq.x = rfma(ad.dw[k], rs.x, Dq.x);
                    Dq.y = rfma(ad.dw[k], rs.y, Dq.y);
                }
            }
        }
        const R sg = m ? (R)-1 : (R)1;               // a mirrored column holds conjugated values
        const R wc = ac.w[j];
        val.x = rfma(wc, A.x, val.x);
        val.y = rfma(sg * wc, A.y, val.y);
        if (WITH_DERIV) {
            g_c.x = rfma(ac.dw[j], A.x, g_c.x);
            g_c.y = rfma(sg * ac.dw[j], A.y, g_c.y);
            g_r.x = rfma(wc, Bq.x, g_r.x);
            g_r.y = rfma(sg * wc, Bq.y, g_r.y);
            g_d.x = rfma(wc, Dq.x, g_d.x);
            g_d.y = rfma(sg * wc, Dq.y, g_d.y);
        }
    }
    }
}


// One lane's share of a cooperative gather: column tap q of every footprint row of the pixel at
// (pc, pr, pd).  Returns the lane's column weight and its derivative (wc, dwc), whether the
// column is a Friedel mate (m: its values are conjugates), and the sums over the footprint's rows
// and planes of the column's voxels: A (value weights), Bq (row-derivative weights), Dq
// (plane-derivative weights).
template <int DIM, bool CUBIC, bool WITH_DERIV, typename R>
__device__ __forceinline__ void coop_column_sums(const SliceGeom& g, const C2<R>* __restrict__ vol,
                                                 R pc, R pr, R pd, int q, R& wc, R& dwc, bool& m,
                                                 C2<R>& A, C2<R>& Bq, C2<R>& Dq) {
    constexpr int T = CUBIC ? 4 : 2;
    constexpr int TD = (DIM == 3) ? T : 1;
    const int plane_stride = g.R * g.Rh;
    AxisWeights<R, T> ar;
    axis_weights<T, WITH_DERIV>(pr, ar);
    // plane weights are formed one at a time inside the loop below (each is used once)
    const R fld = (DIM == 3) ? rfloor(pd) : (R)0;
    const R fd = pd - fld;
    const int dbase = (int)fld - (CUBIC ? 1 : 0);
    // this lane's column tap
    const R flc = rfloor(pc);
    const R fc = pc - flc;
    const int cbase = CUBIC ? (int)flc - 1 : (int)flc;
    const int col = gather_col<CUBIC>(g, cbase + q, m);
    dwc = 0.f;
    if constexpr (CUBIC) {
        R w4[4];
        cubic_weights(fc, w4);
        wc = q == 0 ? w4[0] : q == 1 ? w4[1] : q == 2 ? w4[2] : w4[3];
        if (WITH_DERIV) {
            R d4[4];
            cubic_dweights(fc, d4);
            dwc = q == 0 ? d4[0] : q == 1 ? d4[1] : q == 2 ? d4[2] : d4[3];
        }
    } else {
        wc = q ? fc : 1.f - fc;
        dwc = q ? 1.f : -1.f;
    }
    int rowcol[T];
#pragma unroll
    for (int i = 0; i < T; ++i) rowcol[i] = gather_line<CUBIC>(g, ar.base + i, m) * g.Rh + col;

    A = make2<R>(0.f, 0.f);
    Bq = A;
    Dq = A;
    if constexpr (sizeof(R) == 4 && !WITH_DERIV) {
        // fp32, value only: both components of a complex sum advance in one packed fused
        // multiply-add (fma.rn.f32x2, the same two roundings as two scalar ones), which halves the
        // arithmetic instructions of the gather (measured on B200: cubic forward projection -1 % in
        // 3D, -3.4 % in 2D; with the derivative sums beside it the packed form was 5-20 % slower, so
        // those keep scalar operations)
        unsigned long long w2[T], dw2[T], A2 = 0ull, B2 = 0ull, D2 = 0ull;
#pragma unroll
        for (int i = 0; i < T; ++i) {
            w2[i] = pack2(ar.w[i], ar.w[i]);
            dw2[i] = WITH_DERIV ? pack2(ar.dw[i], ar.dw[i]) : 0ull;
        }
#pragma unroll
        for (int k = 0; k < TD; ++k) {
            const float2* __restrict__ pl = (const float2*)vol + ((DIM == 3) ? gather_line<CUBIC>(g, dbase + k, m) * plane_stride : 0);
            unsigned long long rs2 = 0ull, rds2 = 0ull;
#pragma unroll
            for (int i = 0; i < T; ++i) {
                const float2 v = __ldg(pl + rowcol[i]);
                const unsigned long long v2 = pack2(v.x, v.y);
                rs2 = fma2(w2[i], v2, rs2);
                if (WITH_DERIV) rds2 = fma2(dw2[i], v2, rds2);
            }
            float wd = 1.f, dwd = 0.f;
            if (DIM == 3) {
                if constexpr (CUBIC) {
                    wd = k == 0 ? cubic_weight_k<0>((float)fd) : k == 1 ? cubic_weight_k<1>((float)fd) : k == 2 ? cubic_weight_k<2>((float)fd) : cubic_weight_k<3>((float)fd);
                    if (WITH_DERIV)
                        dwd = k == 0 ? cubic_dweight_k<0>((float)fd) : k == 1 ? cubic_dweight_k<1>((float)fd) : k == 2 ? cubic_dweight_k<2>((float)fd) : cubic_dweight_k<3>((float)fd);
                } else {
                    wd = k ? (float)fd : 1.f - (float)fd;
                    dwd = k ? 1.f : -1.f;
                }
            }
            const unsigned long long wd2 = pack2(wd, wd);
            A2 = fma2(wd2, rs2, A2);
            if (WITH_DERIV) {
                B2 = fma2(wd2, rds2, B2);
                if (DIM == 3) D2 = fma2(pack2(dwd, dwd), rs2, D2);
            }
        }
        float ax, ay, bx, by, dx, dy;
        unpack2(A2, ax, ay);
        unpack2(B2, bx, by);
        unpack2(D2, dx, dy);
        A = make2<R>(ax, ay);
        Bq = make2<R>(bx, by);
        Dq = make2<R>(dx, dy);
    } else {
#pragma unroll
    for (int k = 0; k < TD; ++k) {
        const C2<R>* __restrict__ pl = vol + ((DIM == 3) ? gather_line<CUBIC>(g, dbase + k, m) * plane_stride : 0);
        C2<R> rs = make2<R>(0.f, 0.f), rds = rs;
#pragma unroll
        for (int i = 0; i < T; ++i) {
            const C2<R> v = __ldg(pl + rowcol[i]);
            rs.x = rfma(ar.w[i], v.x, rs.x);
            rs.y = rfma(ar.w[i], v.y, rs.y);
            if (WITH_DERIV) {
                rds.x = rfma(ar.dw[i], v.x, rds.x);
                rds.y = rfma(ar.dw[i], v.y, rds.y);
            }
        }
        R wd = 1.f, dwd = 0.f;
        if (DIM == 3) {
            if constexpr (CUBIC) {
                wd = k == 0 ? cubic_weight_k<0>(fd) : k == 1 ? cubic_weight_k<1>(fd) : k == 2 ? cubic_weight_k<2>(fd) : cubic_weight_k<3>(fd);
                if (WITH_DERIV)
                    dwd = k == 0 ? cubic_dweight_k<0>(fd) : k == 1 ? cubic_dweight_k<1>(fd) : k == 2 ? cubic_dweight_k<2>(fd) : cubic_dweight_k<3>(fd);
            } else {
                wd = k ? fd : 1.f - fd;
                dwd = k ? 1.f : -1.f;
            }
        }
        A.x = rfma(wd, rs.x, A.x);
        A.y = rfma(wd, rs.y, A.y);
        if (WITH_DERIV) {
            Bq.x = rfma(wd, rds.x, Bq.x);
            Bq.y = rfma(wd, rds.y, Bq.y);
            if (DIM == 3) {
                Dq.x = rfma(dwd, rs.x, Dq.x);
                Dq.y = rfma(dwd, rs.y, Dq.y);
            }
        }
    }
    }
}

// Cooperative separable interpolation of a complex half-volume, optionally with the spatial
// derivatives (d/dc, d/dr, d/dd).  The T lanes of a group (T = 2 linear, 4 cubic; groups
// are aligned runs of lanes, whose pixels are T consecutive columns of one slice row) work
// on ONE pixel at a time: lane q fetches column tap q of every footprint row, so that a
// group's loads of one row are T adjacent voxels (one or two 32-byte sectors) instead of T
// separate requests by one lane.  Measured on B200 (cubic, box 256): ~14 instead of ~30
// sectors per warp request and 1.57x the throughput of one-lane-per-pixel gathers.
// Each lane keeps the partial sums of its column, weights them and the group adds them up
// with shuffles.  Because lane q only ever touches column q, the Friedel mirror of that
// column (which decides rows and planes, see gather_line) is a per-lane constant and the
// footprints that straddle c = 0 need no special case.
// MUST be called by all 32 lanes of the warp; lanes without a pixel pass valid_own = false.
// vol points at the batch item.
template <int DIM, bool CUBIC, bool WITH_DERIV, typename R>
__device__ __forceinline__ void interpolate_coop(const SliceGeom& g, const C2<R>* __restrict__ vol,
                                                 const PixelT<R>& px, bool valid_own, C2<R>& val,
                                                 C2<R>& g_c, C2<R>& g_r, C2<R>& g_d) {
    constexpr int T = CUBIC ? 4 : 2;
    constexpr unsigned kFull = 0xffffffffu;
    const int lane = threadIdx.x & 31;
    const int q = lane & (T - 1);
    val = make2<R>(0.f, 0.f);
    g_c = g_r = g_d = val;

    // the loop over the group's pixels stays rolled: its body holds T*T unrolled taps, and T
    // copies of it overflow the instruction cache (seen as no_instruction stalls)
#pragma unroll 1
    for (int s = 0; s < T; ++s) {
        const int src = (lane & ~(T - 1)) | s;
        const R pc = __shfl_sync(kFull, px.c, src);
        const R pr = __shfl_sync(kFull, px.r, src);
        const R pd = (DIM == 3) ? __shfl_sync(kFull, px.d, src) : 0.f;
        const bool valid = __shfl_sync(kFull, (int)valid_own, src) != 0;

        C2<R> cv = make2<R>(0.f, 0.f), cgc = cv, cgr = cv, cgd = cv;
        if (valid) {
            R wc, dwc;
            bool m;
            C2<R> A, Bq, Dq;
            coop_column_sums<DIM, CUBIC, WITH_DERIV>(g, vol, pc, pr, pd, q, wc, dwc, m, A, Bq, Dq);
            const R sg = m ? -1.f : 1.f;          // a mirrored column holds conjugated values
            cv = make2<R>(wc * A.x, sg * wc * A.y);
            if (WITH_DERIV) {
                cgc = make2<R>(dwc * A.x, sg * dwc * A.y);
                cgr = make2<R>(wc * Bq.x, sg * wc * Bq.y);
                cgd = make2<R>(wc * Dq.x, sg * wc * Dq.y);
            }
        }
#pragma unroll
        for (int o = 1; o < T; o <<= 1) {
            cv.x += __shfl_xor_sync(kFull, cv.x, o);
            cv.y += __shfl_xor_sync(kFull, cv.y, o);
            if (WITH_DERIV) {
                cgc.x += __shfl_xor_sync(kFull, cgc.x, o);
                cgc.y += __shfl_xor_sync(kFull, cgc.y, o);
                cgr.x += __shfl_xor_sync(kFull, cgr.x, o);
                cgr.y += __shfl_xor_sync(kFull, cgr.y, o);
                if (DIM == 3) {
                    cgd.x += __shfl_xor_sync(kFull, cgd.x, o);
                    cgd.y += __shfl_xor_sync(kFull, cgd.y, o);
                }
            }
        }
        if (q == s) {
            val = cv;
            g_c = cgc;
            g_r = cgr;
            g_d = cgd;
        }
    }
}

// What the backward of the forward projection needs from the gather, as real scalars: with
// u = grad * conj(phase) of a pixel and the interpolated value v and its derivatives there,
//   dots[0..2] = Re(u * conj(dv/dc)), Re(u * conj(dv/dr)), Re(u * conj(dv/dd))   (rotation gradient)
//   dots[3]    = Im(u * conj(v))                                                  (shift gradient)
// All four are linear in the gathered voxels, so in the cooperative form every lane of a group
// dots ITS column's partial sums with the pixel's u (sent along with the position) and the group
// adds four scalars instead of eight complex components; only four registers per pixel outlive
// the gather.  MUST be called by all 32 lanes of the warp.
// WITH_VALUE (the backward of back-projection, which also writes the interpolated value out): the
// complex value v comes back in `value` as well (two more scalars through the group's reduction),
// and dots[3] is then formed from it by the owner instead of being reduced.
template <int DIM, bool CUBIC, bool NEED_ROT, bool WITH_VALUE = false, typename R>
__device__ __forceinline__ void gather_pose_dots(const SliceGeom& g, const C2<R>* __restrict__ vol,
                                                 const PixelT<R>& px, bool valid_own, C2<R> u_own,
                                                 R (&dots)[4], C2<R>* value = nullptr) {
    constexpr int T = CUBIC ? 4 : 2;
    constexpr unsigned kFull = 0xffffffffu;
#pragma unroll
    for (int v = 0; v < 4; ++v) dots[v] = 0.f;
    if (WITH_VALUE) *value = make2<R>(0.f, 0.f);
    if (!(CUBIC || (DIM == 3 && g.sparse_samples))) {            // warp-uniform: one lane per pixel
        if (valid_own) {
            C2<R> val, gc, gr, gd;
            interpolate_lane<DIM, CUBIC, NEED_ROT>(g, vol, px, val, gc, gr, gd);
            if (NEED_ROT) {
                dots[0] = u_own.x * gc.x + u_own.y * gc.y;
                dots[1] = u_own.x * gr.x + u_own.y * gr.y;
                if (DIM == 3) dots[2] = u_own.x * gd.x + u_own.y * gd.y;
            }
            dots[3] = u_own.y * val.x - u_own.x * val.y;
            if (WITH_VALUE) *value = val;
        }
        return;
    }
    const int lane = threadIdx.x & 31;
    const int q = lane & (T - 1);
#pragma unroll 1
    for (int s = 0; s < T; ++s) {
        const int src = (lane & ~(T - 1)) | s;
        const R pc = __shfl_sync(kFull, px.c, src);
        const R pr = __shfl_sync(kFull, px.r, src);
        const R pd = (DIM == 3) ? __shfl_sync(kFull, px.d, src) : 0.f;
        const R ux = __shfl_sync(kFull, u_own.x, src);
        const R uy = __shfl_sync(kFull, u_own.y, src);
        const bool valid = __shfl_sync(kFull, (int)valid_own, src) != 0;
        R part[4] = {0.f, 0.f, 0.f, 0.f};
        C2<R> cv = make2<R>(0.f, 0.f);
        if (valid) {
            R wc, dwc;
            bool m;
            C2<R> A, Bq, Dq;
            coop_column_sums<DIM, CUBIC, NEED_ROT>(g, vol, pc, pr, pd, q, wc, dwc, m, A, Bq, Dq);
            const R uys = m ? -uy : uy;                      // a mirrored column holds conjugated values
            if (NEED_ROT) {
                part[0] = dwc * (ux * A.x + uys * A.y);
                part[1] = wc * (ux * Bq.x + uys * Bq.y);
                if (DIM == 3) part[2] = wc * (ux * Dq.x + uys * Dq.y);
            }
            if (WITH_VALUE) cv = make2<R>(wc * A.x, (m ? -wc : wc) * A.y);
            else part[3] = wc * (uy * A.x - (m ? -ux : ux) * A.y);
        }
#pragma unroll
        for (int o = 1; o < T; o <<= 1) {
#pragma unroll
            for (int v = 0; v < 4; ++v)
                if ((v < 3 && NEED_ROT && (v < 2 || DIM == 3)) || (v == 3 && !WITH_VALUE)) part[v] += __shfl_xor_sync(kFull, part[v], o);
            if (WITH_VALUE) {
                cv.x += __shfl_xor_sync(kFull, cv.x, o);
                cv.y += __shfl_xor_sync(kFull, cv.y, o);
            }
        }
        if (q == s) {
#pragma unroll
            for (int v = 0; v < 4; ++v) dots[v] = part[v];
            if (WITH_VALUE) {
                *value = cv;
                dots[3] = u_own.y * cv.x - u_own.x * cv.y;
            }
        }
    }
}

// Gather used by the kernels: lane groups for cubic footprints, one lane per pixel for linear.
// MUST be called by all 32 lanes of the warp (lanes without a pixel pass valid = false).
template <int DIM, bool CUBIC, bool WITH_DERIV, typename R>
__device__ __forceinline__ void interpolate_any(const SliceGeom& g, const C2<R>* __restrict__ vol,
                                                const PixelT<R>& px, bool valid, C2<R>& val,
                                                C2<R>& g_c, C2<R>& g_r, C2<R>& g_d) {
    // measured on B200: cubic always gains from lane groups; linear gains only in 3D when the
    // samples are sparse (oversampling >= 1.5, neighbouring pixels 2 voxels apart), otherwise the
    // shuffles cost more than the saved L1 traffic
    if (CUBIC || (DIM == 3 && g.sparse_samples)) {          // warp-uniform
        interpolate_coop<DIM, CUBIC, WITH_DERIV>(g, vol, px, valid, val, g_c, g_r, g_d);
    } else {
        val = make2<R>(0.f, 0.f);
        g_c = g_r = g_d = val;
        if (valid) interpolate_lane<DIM, CUBIC, WITH_DERIV>(g, vol, px, val, g_c, g_r, g_d);
    }
}

// ---- scatter addressing (taps outside the stored half-volume are dropped) ---------------
// reference: csrc/cpu/common/projection_utils.h:414-493.

// Index of signed row / plane coordinate r for a (non-)mirrored tap, or -1 when dropped.
__host__ __device__ __forceinline__ int scatter_line(const SliceGeom& g, int r, bool mirrored) {
    if (mirrored) r = -r;                          // INT_MIN stays INT_MIN, which the range test drops
    if (r > g.half || r < -g.half + 1) return -1;
    return r < 0 ? r + g.R : r;
}

// Stored column of signed column c (Friedel mirror for c < 0; `mirrored` says so), or -1 when
// the tap is dropped.  The range test comes BEFORE the negation: a sample position at or below
// -2^31 saturates to INT_MIN, which negation leaves negative.
__host__ __device__ __forceinline__ int scatter_col(const SliceGeom& g, int c, bool& mirrored) {
    mirrored = c < 0;
    if (c <= -g.Rh || c >= g.Rh) return -1;
    return mirrored ? -c : c;
}

__device__ __forceinline__ void red_add_v2(float2* addr, float a, float b) {
    asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(addr), "f"(a), "f"(b) : "memory");
}
__device__ __forceinline__ void red_add(float* addr, float a) {
    asm volatile("red.global.add.f32 [%0], %1;" ::"l"(addr), "f"(a) : "memory");
}
__device__ __forceinline__ void red_add(double* addr, double a) {
    asm volatile("red.global.add.f64 [%0], %1;" ::"l"(addr), "d"(a) : "memory");
}
__device__ __forceinline__ void red_add_v2(double2* addr, double a, double b) {   // no vector form for f64
    red_add(&addr->x, a);
    red_add(&addr->y, b);
}

__device__ __forceinline__ void red_add_v4(float4* addr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
// The same with an L2 eviction priority: lines written this way are the last to be evicted.  The
// slab-ordered scatter uses them so that its slab of planes holds its place in L2 against the
// slices streaming through (measured on B200: 19.4 -> 18.8 ms per 8,192 slices of 400x201 into
// box 800; no effect on the kernels whose volume fits L2, which keep the plain forms).
__device__ __forceinline__ unsigned long long l2_keep_policy() {
    unsigned long long policy;
    asm("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ void red_add_v2_keep(float2* addr, float a, float b, unsigned long long policy) {
    asm volatile("red.global.add.L2::cache_hint.v2.f32 [%0], {%1, %2}, %3;" ::"l"(addr), "f"(a), "f"(b), "l"(policy) : "memory");
}
__device__ __forceinline__ void red_add_keep(float* addr, float a, unsigned long long policy) {
    asm volatile("red.global.add.L2::cache_hint.f32 [%0], %1, %2;" ::"l"(addr), "f"(a), "l"(policy) : "memory");
}
__device__ __forceinline__ void red_add_v2_keep(double2* addr, double a, double b, unsigned long long) { red_add_v2(addr, a, b); }
__device__ __forceinline__ void red_add_keep(double* addr, double a, unsigned long long) { red_add(addr, a); }
__device__ __forceinline__ void red_add_v4_keep(float4* addr, float a, float b, float c, float d, unsigned long long policy) {
    asm volatile("red.global.add.L2::cache_hint.v4.f32 [%0], {%1, %2, %3, %4}, %5;" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d), "l"(policy) : "memory");
}

// Cooperative scatter of a complex value (and, when WEIGHTS, of wval * |tap weight|) to the
// 2^dim / 4^dim taps around a pixel's sample position.  The T lanes of a group (T = 2 linear,
// 4 cubic) distribute ONE pixel at a time; lane q owns column tap q of every footprint row,
// so the group's reductions of one row go to T adjacent voxels (one or two 32-byte sectors).
// The L2 retires reductions per sector and instruction, so fewer sectors per instruction is
// what makes this faster than one lane per pixel (measured on B200, box 256: linear 1.6x,
// cubic 2.4x).
// Tap rules (reference: csrc/cpu/common/projection_utils.h:170-300, 414-493): Friedel mirror
// for c < 0 with conjugation, taps outside the stored half-volume are dropped, zero-weight
// taps are skipped; WITH_DUP also adds the conjugate to the Friedel partner of taps on the
// c == 0 plane (back-projection does; the gradient of the forward projection does not).
// INTERLEAVED: vol4 is a 16-byte-per-voxel (re, im, w, 0) accumulation volume, so that data
// and weight of a tap go out as ONE red.global.add.v4.f32; otherwise vol (complex) and, when
// WEIGHTS, wvol (R) are reduced into directly (v2 + scalar reduction).
// MUST be called by all 32 lanes of the warp; lanes without a pixel pass valid_own = false.
// SLAB: only reductions that LAND in planes with signed coordinate in [z_lo, z_hi) are issued
// (a tap by the plane it lands in after the mirror, the Friedel duplicate of a c == 0 tap by the
// plane of its partner), so a pass of the slab-ordered back-projection writes nothing outside the
// planes it owns and, over all passes, every reduction is issued exactly once.
template <int DIM, bool CUBIC, bool WEIGHTS, bool WITH_DUP, bool INTERLEAVED, bool SLAB = false, typename R>
__device__ __forceinline__ void scatter_coop(const SliceGeom& g, C2<R>* __restrict__ vol,
                                             NoDeduce<R>* __restrict__ wvol, float4* __restrict__ vol4,
                                             const PixelT<R>& px, bool valid_own, C2<R> v_own,
                                             NoDeduce<R> w_own, int z_lo = 0, int z_hi = 0) {
    constexpr int T = CUBIC ? 4 : 2;
    constexpr int TD = (DIM == 3) ? T : 1;
    constexpr unsigned kFull = 0xffffffffu;
    const int lane = threadIdx.x & 31;
    const int q = lane & (T - 1);
    const int plane_stride = g.R * g.Rh;
#pragma unroll 1
    for (int s = 0; s < T; ++s) {
        const int src = (lane & ~(T - 1)) | s;
        const R pc = __shfl_sync(kFull, px.c, src);
        const R pr = __shfl_sync(kFull, px.r, src);
        const R pd = (DIM == 3) ? __shfl_sync(kFull, px.d, src) : 0.f;
        const R vx = __shfl_sync(kFull, v_own.x, src);
        const R vy = __shfl_sync(kFull, v_own.y, src);
        const R wval = WEIGHTS ? __shfl_sync(kFull, w_own, src) : 0.f;
        const bool valid = __shfl_sync(kFull, (int)valid_own, src) != 0;
        if (!valid) continue;
        // this lane's column tap
        const R flc = rfloor(pc);
        const R fc = pc - flc;
        int c = (CUBIC ? (int)flc - 1 : (int)flc) + q;
        R wc;
        if constexpr (CUBIC) {
            R w4[4];
            cubic_weights(fc, w4);
            wc = q == 0 ? w4[0] : q == 1 ? w4[1] : q == 2 ? w4[2] : w4[3];
        } else {
            wc = q ? fc : 1.f - fc;
        }
        bool m;
        c = scatter_col(g, c, m);
        if (c < 0 || wc == 0.f) continue;
        const R sgn = m ? -1.f : 1.f;
        AxisWeights<R, T> ar, ad;
        axis_weights<T, false>(pr, ar);
        if (DIM == 3) axis_weights<T, false>(pd, ad);
#pragma unroll
        for (int k = 0; k < TD; ++k) {
            int dl = 0;
            R wd = 1.f;
            bool tap_here = true, dup_here = true;      // SLAB: which of the two land in [z_lo, z_hi)
            if (DIM == 3) {
                if (SLAB) {
                    const int sd = m ? -(ad.base + k) : ad.base + k;
                    tap_here = sd >= z_lo && sd < z_hi;
                    const int sp = (sd == g.half) ? sd : -sd;      // plane R/2 is its own partner
                    dup_here = WITH_DUP && c == 0 && sp >= z_lo && sp < z_hi;
                    if (!tap_here && !dup_here) continue;
                }
                dl = scatter_line(g, ad.base + k, m);
                wd = ad.w[k];
                if (dl < 0 || wd == 0.f) continue;
            }
#pragma unroll
            for (int i = 0; i < T; ++i) {
                const int rl = scatter_line(g, ar.base + i, m);
                const R wr = ar.w[i];
                if (rl < 0 || wr == 0.f) continue;
                const R w = wd * wr * wc;
                const int off = dl * plane_stride + rl * g.Rh + c;
                const R re = vx * w, im = vy * w * sgn;
                const R fw = WEIGHTS ? wval * rabs(w) : 0.f;
                if (!SLAB || tap_here) {
                    if (INTERLEAVED) {
                        if (SLAB) red_add_v4_keep(vol4 + off, re, im, fw, 0.f, l2_keep_policy());
                        else red_add_v4(vol4 + off, re, im, fw, 0.f);
                    } else if (SLAB) {
                        red_add_v2_keep(vol + off, re, im, l2_keep_policy());
                        if (WEIGHTS) red_add_keep(wvol + off, fw, l2_keep_policy());
                    } else {
                        red_add_v2(vol + off, re, im);
                        if (WEIGHTS) red_add(wvol + off, fw);
                    }
                }
                if (WITH_DUP && c == 0 && (!SLAB || dup_here)) {
                    // Friedel partner (-d, -r, 0); skipped when it is the same voxel
                    const int rl2 = (rl == 0) ? 0 : g.R - rl;
                    const int dl2 = (DIM == 3) ? ((dl == 0) ? 0 : g.R - dl) : 0;
                    if (rl2 != rl || dl2 != dl) {
                        const int off2 = dl2 * plane_stride + rl2 * g.Rh;
                        if (INTERLEAVED) {
                            if (SLAB) red_add_v4_keep(vol4 + off2, re, -im, fw, 0.f, l2_keep_policy());
                            else red_add_v4(vol4 + off2, re, -im, fw, 0.f);
                        } else if (SLAB) {
                            red_add_v2_keep(vol + off2, re, -im, l2_keep_policy());
                            if (WEIGHTS) red_add_keep(wvol + off2, fw, l2_keep_policy());
                        } else {
                            red_add_v2(vol + off2, re, -im);
                            if (WEIGHTS) red_add(wvol + off2, fw);
                        }
                    }
                }
            }
        }
    }
}

// Real-valued tri/bi-linear read of the weight-gradient volume: Friedel mirror without
// conjugation, zero outside.  reference: csrc/cpu/3d/backprojection_2d_to_3d_kernels.cpp:466-515
template <int DIM, typename R>
__device__ __forceinline__ R gather_weight_grad(const SliceGeom& g, const R* __restrict__ wv,
                                                    const PixelT<R>& px) {
    AxisWeights<R, 2> ac, ar, ad;
    axis_weights<2, false>(px.c, ac);
    axis_weights<2, false>(px.r, ar);
    if (DIM == 3) axis_weights<2, false>(px.d, ad);
    const int plane_stride = g.R * g.Rh;
    R acc = 0.f;
#pragma unroll
    for (int k = 0; k < (DIM == 3 ? 2 : 1); ++k) {
        R pk = 0.f;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            R ri = 0.f;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                bool m;
                const int c = scatter_col(g, ac.base + j, m);
                R q = 0.f;
                const int rl = scatter_line(g, ar.base + i, m);
                const int dl = (DIM == 3) ? scatter_line(g, ad.base + k, m) : 0;
                if (c >= 0 && rl >= 0 && dl >= 0) q = __ldg(wv + (dl * plane_stride + rl * g.Rh + c));
                ri = rfma(ac.w[j], q, ri);
            }
            pk = rfma(ar.w[i], ri, pk);
        }
        acc = rfma((DIM == 3) ? ad.w[k] : 1.f, pk, acc);
    }
    return acc;
}

// Sum NV per-thread values over the block and add them to global memory with one atomic
// per value per block.  dst[v] may be nullptr-guarded by the caller through `active`.
template <int NV, typename R>
__device__ __forceinline__ void block_reduce_add(R (&vals)[NV], R* const (&dst)[NV]) {
    __shared__ R red[kWarps][NV];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        R x = vals[v];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
        if (lane == 0) red[warp][v] = x;
    }
    __syncthreads();
    if (threadIdx.x < NV) {
        R x = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) x += red[w][threadIdx.x];
        R* p = dst[threadIdx.x];
        if (p != nullptr && x != 0.f) atomicAdd(p, x);
    }
}

}  // namespace b200proj
