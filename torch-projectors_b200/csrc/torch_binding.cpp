// PyTorch operator layer over the C ABI of include/b200proj.h.
//
// Defines the eight raw operators of warpem/torch-projectors with the reference's schema strings
// (csrc/torch_projectors.cpp:23-36 there) in the namespace torch_projectors_b200, and implements
// them for the CUDA dispatch key: argument checks -> .contiguous() -> allocate outputs -> which
// gradients are wanted (requires_grad of rotations / shifts, as the reference's CUDA wrappers read
// it: csrc/cuda/3d/projection_3d_to_2d_kernels.cu:1066-1067) -> device guard + current stream ->
// one call of the C ABI -> status to TORCH_CHECK.  This is the block a maintainer of the reference
// would put in place of its TORCH_LIBRARY_IMPL(torch_projectors, CUDA, ...) registrations
// (csrc/torch_projectors.cpp:82-95).  No CPU, MPS or autograd-key implementation is registered:
// CPU tensors fail in the dispatcher, and the autograd glue lives in Python as in the reference
// (torch_projectors/ops.py:300-514).
//
// Beyond the reference: complex128 / float64 tensors run on the GPU (the *_f64 entry points);
// the three volume-reading 3D operators exist a second time with a trailing `Tensor? pose_order`
// argument (`*_ordered`), so that a caller can compute the processing order of the slices once
// (`plane_locality_order`) and reuse it in forward, backward and later iterations; shape-only
// implementations for the Meta key let the operators be traced.
#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <atomic>
#include <string>
#include <tuple>

#include "b200proj.h"

namespace {

using at::Tensor;
using OptTensor = c10::optional<Tensor>;

// Volumes (one batch item) at least this large get a locality-preserving processing order of their
// slices when the caller gives none; below it the whole volume stays in the 126 MB L2 and the
// order changes nothing.  Adjustable through the _set_pose_order_thresholds operator.
std::atomic<int64_t> g_order_min_bytes{96ll << 20};
std::atomic<int64_t> g_order_min_poses{64};

inline void status(int rc, const char* op) {
    TORCH_CHECK(rc == B200PROJ_OK, op, ": ", b200proj_last_error(), " (code ", rc, ")");
}

inline int interp_code(const std::string& interpolation) {
    TORCH_CHECK(interpolation == "linear" || interpolation == "cubic", "Supported interpolation methods: 'linear', 'cubic'");
    return interpolation == "cubic" ? B200PROJ_CUBIC : B200PROJ_LINEAR;
}

inline bool is_f64(const Tensor& complex_like) { return complex_like.scalar_type() == at::kComplexDouble; }

inline at::ScalarType real_of(const Tensor& complex_like) { return is_f64(complex_like) ? at::kDouble : at::kFloat; }

void check_complex(const char* name, const Tensor& t, const Tensor* like = nullptr) {
    TORCH_CHECK(t.scalar_type() == at::kComplexFloat || t.scalar_type() == at::kComplexDouble, name, " has dtype ", t.scalar_type(),
                "; the B200 kernels compute in complex64/float32 or complex128/float64 only and there is no CPU fallback for other precisions");
    if (like != nullptr)
        TORCH_CHECK(t.scalar_type() == like->scalar_type(), name, " has dtype ", t.scalar_type(), " but ", like->scalar_type(),
                    " is needed to match the data (mixed precisions are not supported)");
}

void check_real(const char* name, const Tensor& t, const Tensor& like) {
    TORCH_CHECK(t.scalar_type() == at::kFloat || t.scalar_type() == at::kDouble, name, " has dtype ", t.scalar_type(),
                "; the B200 kernels compute in complex64/float32 or complex128/float64 only and there is no CPU fallback for other precisions");
    TORCH_CHECK(t.scalar_type() == real_of(like), name, " has dtype ", t.scalar_type(), " but ", real_of(like), " is needed to match the ",
                like.scalar_type(), " data (mixed precisions are not supported)");
}

struct Poses {
    int64_t P = 0, B_rot = 1, B_shift = 0;
    Tensor rot;
    Tensor shifts;      // undefined when there are none
};

// Shape / device / dtype checks shared by all operators (expanded or sliced pose tensors are legal
// inputs: they are made contiguous here).
Poses check_poses(int dim, const char* what, int64_t B, const Tensor& rotations, const OptTensor& shifts, const Tensor& like) {
    Poses p;
    TORCH_CHECK(rotations.is_cuda(), "Input rotations must be on CUDA device");
    TORCH_CHECK(rotations.dim() == 4 && rotations.size(2) == dim && rotations.size(3) == dim, "Rotations must be (B_rot, P, ", dim, ", ", dim, ")");
    TORCH_CHECK(rotations.device() == like.device(), "rotations must be on the same device as the data");
    check_real("rotations", rotations, like);
    p.B_rot = rotations.size(0);
    p.P = rotations.size(1);
    TORCH_CHECK(p.B_rot == B || p.B_rot == 1, "Batch size of rotations must be 1 or same as ", what);
    p.rot = rotations.contiguous();
    if (shifts.has_value() && shifts->defined()) {
        const Tensor& s = *shifts;
        TORCH_CHECK(s.is_cuda(), "Shifts must be on CUDA device");
        TORCH_CHECK(s.dim() == 3, "Shifts must be (B_shift, P, 2)");
        TORCH_CHECK(s.size(2) == 2, "Shifts must have 2 components (x, y)");
        TORCH_CHECK(s.size(0) == B || s.size(0) == 1, "Batch size of shifts must be 1 or same as ", what);
        TORCH_CHECK(s.size(1) == p.P, "Number of poses in shifts must match rotations");
        TORCH_CHECK(s.scalar_type() == rotations.scalar_type(), "Shifts and rotations must have the same dtype");
        TORCH_CHECK(s.device() == like.device(), "shifts must be on the same device as the data");
        p.shifts = s.contiguous();
        p.B_shift = s.size(0);
    }
    return p;
}

void check_rec(int dim, const Tensor& rec) {
    TORCH_CHECK(rec.dim() == dim + 1, "Reconstruction must have ", dim + 1, " dimensions");
    const int64_t R = rec.size(-2), Rh = rec.size(-1);
    TORCH_CHECK(R % 2 == 0 && Rh == R / 2 + 1, "Reconstruction must be rfft-shaped with an even box (got ", rec.sizes(), ")");
    if (dim == 3) TORCH_CHECK(rec.size(1) == R, "Reconstruction volume must be cubic (depth == height)");
}

inline double cutoff_of(const c10::optional<double>& cutoff, int64_t N) {
    // default: Nyquist radius of the projection (reference: projection_3d_to_2d_kernels.cu:892)
    return cutoff.has_value() ? *cutoff : (double)N / 2.0;
}

template <typename T>
inline const T* cptr(const Tensor& t) { return t.defined() ? static_cast<const T*>(t.data_ptr()) : nullptr; }
template <typename T>
inline T* mptr(Tensor& t) { return t.defined() ? static_cast<T*>(t.data_ptr()) : nullptr; }

inline void* current_stream(const Tensor& t) { return (void*)c10::cuda::getCurrentCUDAStream(t.get_device()).stream(); }

Tensor empty_real0(const Tensor& like, at::ScalarType dt) { return at::empty({0}, like.options().dtype(dt)); }

// ---- processing order of the slices -------------------------------------------------------------
// int32 [B*P] order for the volume-reading 3D operators (b200proj_pose_order_3d).
Tensor plane_locality_order(const Tensor& rotations, int64_t batch) {
    TORCH_CHECK(rotations.is_cuda(), "Input rotations must be on CUDA device");
    TORCH_CHECK(rotations.dim() == 4 && rotations.size(2) == 3 && rotations.size(3) == 3, "Rotations must be (B_rot, P, 3, 3)");
    TORCH_CHECK(rotations.scalar_type() == at::kFloat || rotations.scalar_type() == at::kDouble, "rotations must be float32 or float64");
    TORCH_CHECK(batch >= 1 && (rotations.size(0) == 1 || rotations.size(0) == batch), "Batch size of rotations must be 1 or same as reconstruction");
    const Tensor rot = rotations.contiguous();
    const int64_t P = rot.size(1);
    c10::cuda::CUDAGuard guard(rot.device());
    Tensor order = at::empty({batch * P}, rot.options().dtype(at::kInt));
    if (order.numel() == 0) return order;
    const int rc = rot.scalar_type() == at::kDouble
        ? b200proj_pose_order_3d_f64(cptr<double>(rot), batch, rot.size(0), P, mptr<int32_t>(order), current_stream(rot))
        : b200proj_pose_order_3d(cptr<float>(rot), batch, rot.size(0), P, mptr<int32_t>(order), current_stream(rot));
    status(rc, "plane_locality_order");
    return order;
}

// The order an operator uses: the caller's (checked), or one made here when the volume is large.
Tensor resolve_order(int dim, const Tensor& vol, int64_t B, const Poses& p, const OptTensor& given) {
    if (dim != 3) return Tensor();
    if (given.has_value() && given->defined()) {
        const Tensor& o = *given;
        if (o.numel() == 0) return Tensor();          // an empty tensor = natural order, nothing computed
        TORCH_CHECK(o.is_cuda() && o.device() == vol.device() && o.scalar_type() == at::kInt && o.dim() == 1 && o.numel() == B * p.P,
                    "pose_order must be an int32 CUDA tensor of B*P = ", B * p.P, " entries on the device of the data");
        return o.contiguous();
    }
    if (p.P < g_order_min_poses.load() || vol[0].numel() * (int64_t)vol.element_size() < g_order_min_bytes.load()) return Tensor();
    return plane_locality_order(p.rot, B);
}

// ---- forward projection ---------------------------------------------------------------------------
Tensor project_forw(int dim, const Tensor& reconstruction, const Tensor& rotations, const OptTensor& shifts, at::IntArrayRef output_shape,
                    const std::string& interpolation, double oversampling, const c10::optional<double>& cutoff, const OptTensor& pose_order) {
    TORCH_CHECK(reconstruction.is_cuda(), "Input reconstruction must be on CUDA device");
    TORCH_CHECK(reconstruction.is_complex(), "Reconstruction must be a complex tensor");
    const int interp = interp_code(interpolation);
    check_rec(dim, reconstruction);
    check_complex("reconstruction", reconstruction);
    const int64_t B = reconstruction.size(0), R = reconstruction.size(-2);
    const Poses p = check_poses(dim, "reconstruction", B, rotations, shifts, reconstruction);
    TORCH_CHECK(output_shape.size() >= 1, "output_shape must have at least one element");
    const int64_t N = output_shape[0];            // only element 0 is used, as in the reference
    TORCH_CHECK(N >= 2 && N % 2 == 0, "Output boxsize ", N, " must be even");
    const Tensor rec = reconstruction.contiguous();
    c10::cuda::CUDAGuard guard(rec.device());
    Tensor out = at::empty({B, p.P, N, N / 2 + 1}, rec.options());
    if (out.numel() == 0) return out;
    Tensor order = resolve_order(dim, rec, B, p, pose_order);
    void* s = current_stream(rec);
    const double cut = cutoff_of(cutoff, N);
    int rc;
    if (is_f64(rec)) {
        rc = dim == 2 ? b200proj_project_2d_forw_f64(cptr<double>(rec), B, R, cptr<double>(p.rot), p.B_rot, cptr<double>(p.shifts), p.B_shift, p.P, N, interp, oversampling, cut, mptr<double>(out), s)
                      : b200proj_project_3d_to_2d_forw_f64(cptr<double>(rec), B, R, cptr<double>(p.rot), p.B_rot, cptr<double>(p.shifts), p.B_shift, p.P, N, interp, oversampling, cut, mptr<double>(out), cptr<int32_t>(order), s);
    } else {
        rc = dim == 2 ? b200proj_project_2d_forw(cptr<float>(rec), B, R, cptr<float>(p.rot), p.B_rot, cptr<float>(p.shifts), p.B_shift, p.P, N, interp, oversampling, cut, mptr<float>(out), s)
                      : b200proj_project_3d_to_2d_forw(cptr<float>(rec), B, R, cptr<float>(p.rot), p.B_rot, cptr<float>(p.shifts), p.B_shift, p.P, N, interp, oversampling, cut, mptr<float>(out), cptr<int32_t>(order), s);
    }
    status(rc, dim == 2 ? "project_2d_forw" : "project_3d_to_2d_forw");
    return out;
}

// ---- backward of forward projection ---------------------------------------------------------------
std::tuple<Tensor, Tensor, Tensor> project_back(int dim, const Tensor& grad_projections, const Tensor& reconstruction, const Tensor& rotations,
                                                const OptTensor& shifts, const std::string& interpolation, double oversampling,
                                                const c10::optional<double>& cutoff, const OptTensor& pose_order) {
    TORCH_CHECK(grad_projections.is_cuda(), "Input grad_projections must be on CUDA device");
    TORCH_CHECK(reconstruction.is_cuda(), "Input reconstruction must be on CUDA device");
    TORCH_CHECK(grad_projections.is_complex(), "Projections must be a complex tensor");
    TORCH_CHECK(reconstruction.is_complex(), "Reconstruction must be a complex tensor");
    const int interp = interp_code(interpolation);
    TORCH_CHECK(grad_projections.dim() == 4, "Projections must be a 4D tensor (B, P, H, W/2+1)");
    check_rec(dim, reconstruction);
    check_complex("reconstruction", reconstruction);
    check_complex("grad_projections", grad_projections, &reconstruction);
    const int64_t B = grad_projections.size(0), P_g = grad_projections.size(1), N = grad_projections.size(2), Nh = grad_projections.size(3);
    TORCH_CHECK(N % 2 == 0 && Nh == N / 2 + 1, "grad_projections must be rfft-shaped with an even box");
    TORCH_CHECK(reconstruction.size(0) == B, "Batch size of grad_projections must match reconstruction");
    const Poses p = check_poses(dim, "reconstruction", B, rotations, shifts, reconstruction);
    TORCH_CHECK(p.P == P_g, "Number of poses in rotations must match grad_projections");
    const bool need_rot = rotations.requires_grad();
    const bool need_shift = p.shifts.defined() && shifts->requires_grad();
    const Tensor gp = grad_projections.contiguous();
    const Tensor rec = reconstruction.contiguous();
    const int64_t R = rec.size(-2);
    c10::cuda::CUDAGuard guard(rec.device());
    Tensor grad_rec = at::empty_like(rec);                 // zero-filled by the library call
    Tensor grad_rot = need_rot ? at::empty_like(p.rot) : Tensor();
    Tensor grad_sh = need_shift ? at::empty_like(p.shifts) : Tensor();
    if (p.P == 0 || gp.numel() == 0) {                     // nothing to launch: pointers of empty tensors are NULL
        grad_rec.zero_();
    } else {
        Tensor order = resolve_order(dim, rec, B, p, pose_order);
        void* s = current_stream(rec);
        const double cut = cutoff_of(cutoff, N);
        int rc;
        if (is_f64(rec)) {
            rc = dim == 2 ? b200proj_project_2d_back_f64(cptr<double>(gp), cptr<double>(rec), B, R, cptr<double>(p.rot), p.B_rot, cptr<double>(p.shifts), p.B_shift, p.P, N, interp, oversampling, cut, mptr<double>(grad_rec), mptr<double>(grad_rot), mptr<double>(grad_sh), s)
                          : b200proj_project_3d_to_2d_back_f64(cptr<double>(gp), cptr<double>(rec), B, R, cptr<double>(p.rot), p.B_rot, cptr<double>(p.shifts), p.B_shift, p.P, N, interp, oversampling, cut, mptr<double>(grad_rec), mptr<double>(grad_rot), mptr<double>(grad_sh), cptr<int32_t>(order), s);
        } else {
            rc = dim == 2 ? b200proj_project_2d_back(cptr<float>(gp), cptr<float>(rec), B, R, cptr<float>(p.rot), p.B_rot, cptr<float>(p.shifts), p.B_shift, p.P, N, interp, oversampling, cut, mptr<float>(grad_rec), mptr<float>(grad_rot), mptr<float>(grad_sh), s)
                          : b200proj_project_3d_to_2d_back(cptr<float>(gp), cptr<float>(rec), B, R, cptr<float>(p.rot), p.B_rot, cptr<float>(p.shifts), p.B_shift, p.P, N, interp, oversampling, cut, mptr<float>(grad_rec), mptr<float>(grad_rot), mptr<float>(grad_sh), cptr<int32_t>(order), s);
        }
        status(rc, dim == 2 ? "project_2d_back" : "project_3d_to_2d_back");
    }
    const at::ScalarType rd = p.rot.scalar_type();
    return std::make_tuple(grad_rec, need_rot ? grad_rot : empty_real0(rec, rd), need_shift ? grad_sh : empty_real0(rec, rd));
}

// ---- forward projection that keeps the pixels' derivatives, and its backward pass --------------------
// (additions; complex64 only: the step of an optimisation over poses needs no second gather of the
// volume in its backward pass, and none of the volume's gradient when the volume is fixed)
std::tuple<Tensor, Tensor> project_forw_saving(int dim, const Tensor& reconstruction, const Tensor& rotations, const OptTensor& shifts,
                                               at::IntArrayRef output_shape, const std::string& interpolation, double oversampling,
                                               const c10::optional<double>& cutoff, const OptTensor& pose_order) {
    TORCH_CHECK(reconstruction.is_cuda(), "Input reconstruction must be on CUDA device");
    TORCH_CHECK(reconstruction.scalar_type() == at::kComplexFloat, "the derivative-saving projection takes complex64 volumes");
    const int interp = interp_code(interpolation);
    check_rec(dim, reconstruction);
    const int64_t B = reconstruction.size(0), R = reconstruction.size(-2);
    const Poses p = check_poses(dim, "reconstruction", B, rotations, shifts, reconstruction);
    TORCH_CHECK(output_shape.size() >= 1, "output_shape must have at least one element");
    const int64_t N = output_shape[0];
    TORCH_CHECK(N >= 2 && N % 2 == 0, "Output boxsize ", N, " must be even");
    const Tensor rec = reconstruction.contiguous();
    c10::cuda::CUDAGuard guard(rec.device());
    Tensor out = at::empty({B, p.P, N, N / 2 + 1}, rec.options());
    Tensor derivs = at::empty({dim, B, p.P, N, N / 2 + 1}, rec.options());
    if (out.numel() == 0) return std::make_tuple(out, derivs);
    Tensor order = resolve_order(dim, rec, B, p, pose_order);
    const double cut = cutoff_of(cutoff, N);
    const int rc = dim == 2
        ? b200proj_project_2d_forw_saving(cptr<float>(rec), B, R, cptr<float>(p.rot), p.B_rot, cptr<float>(p.shifts), p.B_shift, p.P, N, interp,
                                          oversampling, cut, mptr<float>(out), mptr<float>(derivs), current_stream(rec))
        : b200proj_project_3d_to_2d_forw_saving(cptr<float>(rec), B, R, cptr<float>(p.rot), p.B_rot, cptr<float>(p.shifts), p.B_shift, p.P, N, interp,
                                                oversampling, cut, mptr<float>(out), mptr<float>(derivs), cptr<int32_t>(order), current_stream(rec));
    status(rc, dim == 2 ? "project_2d_forw_saving" : "project_3d_to_2d_forw_saving");
    return std::make_tuple(out, derivs);
}

std::tuple<Tensor, Tensor, Tensor> project_back_saved(int dim, const Tensor& grad_projections, const Tensor& projections, const Tensor& derivatives,
                                                      const Tensor& reconstruction, const Tensor& rotations, const OptTensor& shifts,
                                                      const std::string& interpolation, double oversampling, const c10::optional<double>& cutoff,
                                                      const OptTensor& pose_order, bool need_rec_grad) {
    TORCH_CHECK(grad_projections.is_cuda() && reconstruction.is_cuda(), "Inputs must be on CUDA device");
    TORCH_CHECK(grad_projections.scalar_type() == at::kComplexFloat && reconstruction.scalar_type() == at::kComplexFloat,
                "the derivative-saving projection takes complex64 tensors");
    const int interp = interp_code(interpolation);
    TORCH_CHECK(grad_projections.dim() == 4, "Projections must be a 4D tensor (B, P, H, W/2+1)");
    check_rec(dim, reconstruction);
    const int64_t B = grad_projections.size(0), P_g = grad_projections.size(1), N = grad_projections.size(2), Nh = grad_projections.size(3);
    TORCH_CHECK(N % 2 == 0 && Nh == N / 2 + 1, "grad_projections must be rfft-shaped with an even box");
    TORCH_CHECK(reconstruction.size(0) == B, "Batch size of grad_projections must match reconstruction");
    const Poses p = check_poses(dim, "reconstruction", B, rotations, shifts, reconstruction);
    TORCH_CHECK(p.P == P_g, "Number of poses in rotations must match grad_projections");
    TORCH_CHECK(projections.sizes() == grad_projections.sizes() && projections.scalar_type() == at::kComplexFloat && projections.is_cuda(),
                "saved projections must match grad_projections");
    const bool need_rot = rotations.requires_grad();
    // the derivatives are read for the rotation gradient only: without it an empty tensor will do
    TORCH_CHECK((!need_rot && derivatives.numel() == 0) ||
                (derivatives.dim() == 5 && derivatives.size(0) == dim && derivatives.sizes().slice(1) == grad_projections.sizes() &&
                 derivatives.scalar_type() == at::kComplexFloat && derivatives.is_cuda()),
                "saved derivatives must be (dim, B, P, H, W/2+1) complex64");
    const bool need_shift = p.shifts.defined() && shifts->requires_grad();
    const Tensor gp = grad_projections.contiguous();
    const Tensor out = projections.contiguous();
    const Tensor der = derivatives.numel() ? derivatives.contiguous() : Tensor();
    const int64_t R = reconstruction.size(-2);
    c10::cuda::CUDAGuard guard(gp.device());
    Tensor grad_rec = need_rec_grad ? at::empty(reconstruction.sizes(), gp.options()) : Tensor();
    Tensor grad_rot = need_rot ? at::empty_like(p.rot) : Tensor();
    Tensor grad_sh = need_shift ? at::empty_like(p.shifts) : Tensor();
    if (p.P == 0 || gp.numel() == 0) {
        if (need_rec_grad) grad_rec.zero_();
    } else {
        Tensor order = resolve_order(dim, reconstruction, B, p, pose_order);
        const double cut = cutoff_of(cutoff, N);
        const int rc = dim == 2
            ? b200proj_project_2d_back_saved(cptr<float>(gp), cptr<float>(out), cptr<float>(der), B, R, cptr<float>(p.rot), p.B_rot, cptr<float>(p.shifts),
                                             p.B_shift, p.P, N, interp, oversampling, cut, mptr<float>(grad_rec), mptr<float>(grad_rot), mptr<float>(grad_sh),
                                             current_stream(gp))
            : b200proj_project_3d_to_2d_back_saved(cptr<float>(gp), cptr<float>(out), cptr<float>(der), B, R, cptr<float>(p.rot), p.B_rot, cptr<float>(p.shifts),
                                                   p.B_shift, p.P, N, interp, oversampling, cut, mptr<float>(grad_rec), mptr<float>(grad_rot), mptr<float>(grad_sh),
                                                   cptr<int32_t>(order), current_stream(gp));
        status(rc, dim == 2 ? "project_2d_back_saved" : "project_3d_to_2d_back_saved");
    }
    const at::ScalarType rd = p.rot.scalar_type();
    return std::make_tuple(need_rec_grad ? grad_rec : empty_real0(gp, rd), need_rot ? grad_rot : empty_real0(gp, rd),
                           need_shift ? grad_sh : empty_real0(gp, rd));
}

// ---- back-projection ------------------------------------------------------------------------------
std::tuple<Tensor, Tensor> backproject_forw(int dim, const Tensor& projections, const OptTensor& weights_opt, const Tensor& rotations,
                                            const OptTensor& shifts, const std::string& interpolation, double oversampling,
                                            const c10::optional<double>& cutoff) {
    TORCH_CHECK(projections.is_cuda(), "Input projections must be on CUDA device");
    TORCH_CHECK(projections.is_complex(), "Projections must be a complex tensor");
    const int interp = interp_code(interpolation);
    TORCH_CHECK(projections.dim() == 4, "Projections must be (B, P, height, width/2+1)");
    check_complex("projections", projections);
    const int64_t B = projections.size(0), P_p = projections.size(1), N = projections.size(2), Nh = projections.size(3);
    TORCH_CHECK(N % 2 == 0 && Nh == N / 2 + 1, "projections must be rfft-shaped with an even box");
    Tensor weights;
    if (weights_opt.has_value() && weights_opt->defined()) {
        const Tensor& w = *weights_opt;
        TORCH_CHECK(w.is_cuda(), "Weights must be on CUDA device");
        TORCH_CHECK(w.is_floating_point(), "Weights must be a real-valued tensor");
        TORCH_CHECK(w.dim() == 4, "Weights must be (B, P, height, width/2+1)");
        TORCH_CHECK(w.sizes() == projections.sizes(), "Weights and projections must have the same shape");
        check_real("weights", w, projections);
        weights = w.contiguous();
    }
    const Poses p = check_poses(dim, "projections", B, rotations, shifts, projections);
    TORCH_CHECK(p.P == P_p, "Number of poses in rotations must match projections");
    const Tensor proj = projections.contiguous();
    c10::cuda::CUDAGuard guard(proj.device());
    const int64_t R = b200proj_rec_boxsize(N, oversampling);
    std::vector<int64_t> shape = dim == 3 ? std::vector<int64_t>{B, R, R, R / 2 + 1} : std::vector<int64_t>{B, R, R / 2 + 1};
    Tensor data_rec = at::empty(shape, proj.options());     // zero-filled by the call
    Tensor weight_rec = weights.defined() ? at::empty(shape, proj.options().dtype(real_of(proj))) : Tensor();
    if (p.P == 0) {                                         // nothing to launch: pointers of empty tensors are NULL
        data_rec.zero_();
        if (weight_rec.defined()) weight_rec.zero_();
    } else {
        void* s = current_stream(proj);
        const double cut = cutoff_of(cutoff, N);
        int rc;
        if (is_f64(proj)) {
            rc = dim == 2 ? b200proj_backproject_2d_forw_f64(cptr<double>(proj), cptr<double>(weights), B, R, cptr<double>(p.rot), p.B_rot, cptr<double>(p.shifts), p.B_shift, p.P, N, interp, oversampling, cut, mptr<double>(data_rec), mptr<double>(weight_rec), 0, nullptr, 0, s)
                          : b200proj_backproject_2d_to_3d_forw_f64(cptr<double>(proj), cptr<double>(weights), B, R, cptr<double>(p.rot), p.B_rot, cptr<double>(p.shifts), p.B_shift, p.P, N, interp, oversampling, cut, mptr<double>(data_rec), mptr<double>(weight_rec), 0, nullptr, 0, s);
        } else {
            // scratch for the interleaved accumulation path, from the caching allocator (nothing is freed behind the stream)
            const size_t ws_bytes = b200proj_backproject_workspace_bytes(dim, B, R, p.P, N, interp, weights.defined() ? 1 : 0);
            Tensor ws = ws_bytes ? at::empty({(int64_t)ws_bytes}, proj.options().dtype(at::kByte)) : Tensor();
            void* wsp = ws.defined() ? ws.data_ptr() : nullptr;
            rc = dim == 2 ? b200proj_backproject_2d_forw(cptr<float>(proj), cptr<float>(weights), B, R, cptr<float>(p.rot), p.B_rot, cptr<float>(p.shifts), p.B_shift, p.P, N, interp, oversampling, cut, mptr<float>(data_rec), mptr<float>(weight_rec), 0, wsp, ws_bytes, s)
                          : b200proj_backproject_2d_to_3d_forw(cptr<float>(proj), cptr<float>(weights), B, R, cptr<float>(p.rot), p.B_rot, cptr<float>(p.shifts), p.B_shift, p.P, N, interp, oversampling, cut, mptr<float>(data_rec), mptr<float>(weight_rec), 0, wsp, ws_bytes, s);
        }
        status(rc, dim == 2 ? "backproject_2d_forw" : "backproject_2d_to_3d_forw");
    }
    if (!weight_rec.defined()) weight_rec = empty_real0(proj, p.rot.scalar_type());
    return std::make_tuple(data_rec, weight_rec);
}

// ---- backward of back-projection ------------------------------------------------------------------
std::tuple<Tensor, Tensor, Tensor, Tensor> backproject_back(int dim, const Tensor& grad_data_rec, const OptTensor& grad_weight_rec_opt,
                                                            const Tensor& projections, const OptTensor& weights_opt, const Tensor& rotations,
                                                            const OptTensor& shifts, const std::string& interpolation, double oversampling,
                                                            const c10::optional<double>& cutoff, const OptTensor& pose_order) {
    TORCH_CHECK(grad_data_rec.is_cuda(), "Input grad_data_rec must be on CUDA device");
    TORCH_CHECK(projections.is_cuda(), "Input projections must be on CUDA device");
    TORCH_CHECK(grad_data_rec.is_complex(), "grad_data_rec must be a complex tensor");
    TORCH_CHECK(projections.is_complex(), "projections must be a complex tensor");
    const int interp = interp_code(interpolation);
    TORCH_CHECK(grad_data_rec.dim() == dim + 1, dim == 3 ? "grad_data_rec must be (B, D, H, W/2+1)" : "grad_data_rec must be (B, H, W/2+1)");
    TORCH_CHECK(projections.dim() == 4, "projections must be a 4D tensor (B, P, boxsize, boxsize/2+1)");
    check_complex("projections", projections);
    check_complex("grad_data_rec", grad_data_rec, &projections);
    const int64_t B = projections.size(0), P_p = projections.size(1), N = projections.size(2);
    Tensor grad_weight_rec;
    if (grad_weight_rec_opt.has_value() && grad_weight_rec_opt->defined()) {
        const Tensor& gw = *grad_weight_rec_opt;
        TORCH_CHECK(gw.is_cuda(), "grad_weight_rec must be on CUDA device");
        TORCH_CHECK(gw.is_floating_point(), "grad_weight_rec must be a real-valued tensor");
        TORCH_CHECK(gw.sizes() == grad_data_rec.sizes(), "grad_weight_rec and grad_data_rec must have same shape");
        check_real("grad_weight_rec", gw, projections);
        grad_weight_rec = gw.contiguous();
    }
    const int64_t R = b200proj_rec_boxsize(N, oversampling);
    std::vector<int64_t> want = dim == 3 ? std::vector<int64_t>{B, R, R, R / 2 + 1} : std::vector<int64_t>{B, R, R / 2 + 1};
    TORCH_CHECK(grad_data_rec.sizes() == at::IntArrayRef(want), "grad_data_rec shape must match expected reconstruction size");
    const bool has_weights = weights_opt.has_value() && weights_opt->defined();
    if (has_weights) {
        TORCH_CHECK(weights_opt->is_cuda(), "weights must be on CUDA device");
        check_real("weights", *weights_opt, projections);
    }
    const Poses p = check_poses(dim, "projections", B, rotations, shifts, projections);
    TORCH_CHECK(p.P == P_p, "Number of poses in rotations must match projections");
    const bool need_rot = rotations.requires_grad();
    const bool need_shift = p.shifts.defined() && shifts->requires_grad();
    const Tensor gd = grad_data_rec.contiguous();
    const Tensor proj = projections.contiguous();
    c10::cuda::CUDAGuard guard(proj.device());
    const at::ScalarType rd = real_of(proj);
    Tensor grad_proj = at::empty_like(proj);
    Tensor grad_w = has_weights ? at::empty(proj.sizes(), proj.options().dtype(rd)) : Tensor();
    Tensor grad_rot = need_rot ? at::empty_like(p.rot) : Tensor();
    Tensor grad_sh = need_shift ? at::empty_like(p.shifts) : Tensor();
    if (proj.numel() != 0) {
        Tensor order = resolve_order(dim, gd, B, p, pose_order);
        void* s = current_stream(proj);
        const double cut = cutoff_of(cutoff, N);
        int rc;
        if (is_f64(proj)) {
            rc = dim == 2 ? b200proj_backproject_2d_back_f64(cptr<double>(gd), cptr<double>(grad_weight_rec), cptr<double>(proj), B, R, cptr<double>(p.rot), p.B_rot, cptr<double>(p.shifts), p.B_shift, p.P, N, interp, oversampling, cut, mptr<double>(grad_proj), mptr<double>(grad_w), mptr<double>(grad_rot), mptr<double>(grad_sh), s)
                          : b200proj_backproject_2d_to_3d_back_f64(cptr<double>(gd), cptr<double>(grad_weight_rec), cptr<double>(proj), B, R, cptr<double>(p.rot), p.B_rot, cptr<double>(p.shifts), p.B_shift, p.P, N, interp, oversampling, cut, mptr<double>(grad_proj), mptr<double>(grad_w), mptr<double>(grad_rot), mptr<double>(grad_sh), cptr<int32_t>(order), s);
        } else {
            rc = dim == 2 ? b200proj_backproject_2d_back(cptr<float>(gd), cptr<float>(grad_weight_rec), cptr<float>(proj), B, R, cptr<float>(p.rot), p.B_rot, cptr<float>(p.shifts), p.B_shift, p.P, N, interp, oversampling, cut, mptr<float>(grad_proj), mptr<float>(grad_w), mptr<float>(grad_rot), mptr<float>(grad_sh), s)
                          : b200proj_backproject_2d_to_3d_back(cptr<float>(gd), cptr<float>(grad_weight_rec), cptr<float>(proj), B, R, cptr<float>(p.rot), p.B_rot, cptr<float>(p.shifts), p.B_shift, p.P, N, interp, oversampling, cut, mptr<float>(grad_proj), mptr<float>(grad_w), mptr<float>(grad_rot), mptr<float>(grad_sh), cptr<int32_t>(order), s);
        }
        status(rc, dim == 2 ? "backproject_2d_back" : "backproject_2d_to_3d_back");
    }
    const at::ScalarType pd = p.rot.scalar_type();
    return std::make_tuple(grad_proj, grad_w.defined() ? grad_w : empty_real0(proj, pd), need_rot ? grad_rot : empty_real0(proj, pd),
                           need_shift ? grad_sh : empty_real0(proj, pd));
}

// ---- the schema-shaped entry points ----------------------------------------------------------------
using Cut = c10::optional<double>;

Tensor project_2d_forw(const Tensor& rec, const Tensor& rot, const OptTensor& sh, at::IntArrayRef shape, std::string interp, double os, Cut cut) {
    return project_forw(2, rec, rot, sh, shape, interp, os, cut, c10::nullopt);
}
Tensor project_3d_to_2d_forw(const Tensor& rec, const Tensor& rot, const OptTensor& sh, at::IntArrayRef shape, std::string interp, double os, Cut cut) {
    return project_forw(3, rec, rot, sh, shape, interp, os, cut, c10::nullopt);
}
Tensor project_3d_to_2d_forw_ordered(const Tensor& rec, const Tensor& rot, const OptTensor& sh, at::IntArrayRef shape, std::string interp, double os, Cut cut, const OptTensor& order) {
    return project_forw(3, rec, rot, sh, shape, interp, os, cut, order);
}
std::tuple<Tensor, Tensor, Tensor> project_2d_back(const Tensor& g, const Tensor& rec, const Tensor& rot, const OptTensor& sh, std::string interp, double os, Cut cut) {
    return project_back(2, g, rec, rot, sh, interp, os, cut, c10::nullopt);
}
std::tuple<Tensor, Tensor, Tensor> project_3d_to_2d_back(const Tensor& g, const Tensor& rec, const Tensor& rot, const OptTensor& sh, std::string interp, double os, Cut cut) {
    return project_back(3, g, rec, rot, sh, interp, os, cut, c10::nullopt);
}
std::tuple<Tensor, Tensor, Tensor> project_3d_to_2d_back_ordered(const Tensor& g, const Tensor& rec, const Tensor& rot, const OptTensor& sh, std::string interp, double os, Cut cut, const OptTensor& order) {
    return project_back(3, g, rec, rot, sh, interp, os, cut, order);
}
std::tuple<Tensor, Tensor> backproject_2d_forw(const Tensor& proj, const OptTensor& w, const Tensor& rot, const OptTensor& sh, std::string interp, double os, Cut cut) {
    return backproject_forw(2, proj, w, rot, sh, interp, os, cut);
}
std::tuple<Tensor, Tensor> backproject_2d_to_3d_forw(const Tensor& proj, const OptTensor& w, const Tensor& rot, const OptTensor& sh, std::string interp, double os, Cut cut) {
    return backproject_forw(3, proj, w, rot, sh, interp, os, cut);
}
std::tuple<Tensor, Tensor, Tensor, Tensor> backproject_2d_back(const Tensor& gd, const OptTensor& gw, const Tensor& proj, const OptTensor& w, const Tensor& rot, const OptTensor& sh, std::string interp, double os, Cut cut) {
    return backproject_back(2, gd, gw, proj, w, rot, sh, interp, os, cut, c10::nullopt);
}
std::tuple<Tensor, Tensor, Tensor, Tensor> backproject_2d_to_3d_back(const Tensor& gd, const OptTensor& gw, const Tensor& proj, const OptTensor& w, const Tensor& rot, const OptTensor& sh, std::string interp, double os, Cut cut) {
    return backproject_back(3, gd, gw, proj, w, rot, sh, interp, os, cut, c10::nullopt);
}
std::tuple<Tensor, Tensor, Tensor, Tensor> backproject_2d_to_3d_back_ordered(const Tensor& gd, const OptTensor& gw, const Tensor& proj, const OptTensor& w, const Tensor& rot, const OptTensor& sh, std::string interp, double os, Cut cut, const OptTensor& order) {
    return backproject_back(3, gd, gw, proj, w, rot, sh, interp, os, cut, order);
}

std::tuple<Tensor, Tensor> project_2d_forw_saving(const Tensor& rec, const Tensor& rot, const OptTensor& sh, at::IntArrayRef shape, std::string interp, double os, Cut cut) {
    return project_forw_saving(2, rec, rot, sh, shape, interp, os, cut, c10::nullopt);
}
std::tuple<Tensor, Tensor> project_3d_to_2d_forw_saving(const Tensor& rec, const Tensor& rot, const OptTensor& sh, at::IntArrayRef shape, std::string interp, double os, Cut cut, const OptTensor& order) {
    return project_forw_saving(3, rec, rot, sh, shape, interp, os, cut, order);
}
std::tuple<Tensor, Tensor, Tensor> project_2d_back_saved(const Tensor& g, const Tensor& proj, const Tensor& der, const Tensor& rec, const Tensor& rot, const OptTensor& sh,
                                                         std::string interp, double os, Cut cut, bool need_rec) {
    return project_back_saved(2, g, proj, der, rec, rot, sh, interp, os, cut, c10::nullopt, need_rec);
}
std::tuple<Tensor, Tensor, Tensor> project_3d_to_2d_back_saved(const Tensor& g, const Tensor& proj, const Tensor& der, const Tensor& rec, const Tensor& rot, const OptTensor& sh,
                                                               std::string interp, double os, Cut cut, const OptTensor& order, bool need_rec) {
    return project_back_saved(3, g, proj, der, rec, rot, sh, interp, os, cut, order, need_rec);
}

void set_pose_order_thresholds(int64_t min_bytes, int64_t min_poses) {
    g_order_min_bytes.store(min_bytes);
    g_order_min_poses.store(min_poses);
}
std::tuple<int64_t, int64_t> get_pose_order_thresholds() { return std::make_tuple(g_order_min_bytes.load(), g_order_min_poses.load()); }

// ---- shape-only implementations (Meta key): what tracing needs -----------------------------------
Tensor meta_project_forw(const Tensor& rec, const Tensor& rot, const OptTensor&, at::IntArrayRef shape, std::string, double, Cut) {
    TORCH_CHECK(rot.dim() == 4 && shape.size() >= 1, "Rotations must be (B_rot, P, d, d) and output_shape non-empty");
    return at::empty({rec.size(0), rot.size(1), shape[0], shape[0] / 2 + 1}, rec.options());
}
Tensor meta_project_forw_ordered(const Tensor& rec, const Tensor& rot, const OptTensor& sh, at::IntArrayRef shape, std::string i, double os, Cut c, const OptTensor&) {
    return meta_project_forw(rec, rot, sh, shape, i, os, c);
}
std::tuple<Tensor, Tensor, Tensor> meta_project_back(const Tensor&, const Tensor& rec, const Tensor& rot, const OptTensor& sh, std::string, double, Cut) {
    const bool ns = sh.has_value() && sh->defined() && sh->requires_grad();
    return std::make_tuple(at::empty_like(rec), rot.requires_grad() ? at::empty_like(rot) : at::empty({0}, rot.options()),
                           ns ? at::empty_like(*sh) : at::empty({0}, rot.options()));
}
std::tuple<Tensor, Tensor, Tensor> meta_project_back_ordered(const Tensor& g, const Tensor& rec, const Tensor& rot, const OptTensor& sh, std::string i, double os, Cut c, const OptTensor&) {
    return meta_project_back(g, rec, rot, sh, i, os, c);
}
template <int DIM>
std::tuple<Tensor, Tensor> meta_backproject_forw(const Tensor& proj, const OptTensor& w, const Tensor& rot, const OptTensor&, std::string, double os, Cut) {
    TORCH_CHECK(proj.dim() == 4, "Projections must be (B, P, height, width/2+1)");
    const int64_t B = proj.size(0), R = b200proj_rec_boxsize(proj.size(2), os);
    std::vector<int64_t> shape = DIM == 3 ? std::vector<int64_t>{B, R, R, R / 2 + 1} : std::vector<int64_t>{B, R, R / 2 + 1};
    const bool hw = w.has_value() && w->defined();
    return std::make_tuple(at::empty(shape, proj.options()), hw ? at::empty(shape, w->options()) : at::empty({0}, rot.options()));
}
std::tuple<Tensor, Tensor, Tensor, Tensor> meta_backproject_back(const Tensor&, const OptTensor&, const Tensor& proj, const OptTensor& w, const Tensor& rot, const OptTensor& sh, std::string, double, Cut) {
    const bool hw = w.has_value() && w->defined();
    const bool ns = sh.has_value() && sh->defined() && sh->requires_grad();
    return std::make_tuple(at::empty_like(proj), hw ? at::empty(proj.sizes(), w->options()) : at::empty({0}, rot.options()),
                           rot.requires_grad() ? at::empty_like(rot) : at::empty({0}, rot.options()), ns ? at::empty_like(*sh) : at::empty({0}, rot.options()));
}
std::tuple<Tensor, Tensor, Tensor, Tensor> meta_backproject_back_ordered(const Tensor& gd, const OptTensor& gw, const Tensor& proj, const OptTensor& w, const Tensor& rot, const OptTensor& sh, std::string i, double os, Cut c, const OptTensor&) {
    return meta_backproject_back(gd, gw, proj, w, rot, sh, i, os, c);
}
std::tuple<Tensor, Tensor> meta_project_forw_saving(const Tensor& rec, const Tensor& rot, const OptTensor& sh, at::IntArrayRef shape, std::string i, double os, Cut c, const OptTensor&) {
    Tensor out = meta_project_forw(rec, rot, sh, shape, i, os, c);
    return std::make_tuple(out, at::empty({3, out.size(0), out.size(1), out.size(2), out.size(3)}, out.options()));
}
std::tuple<Tensor, Tensor> meta_project_2d_forw_saving(const Tensor& rec, const Tensor& rot, const OptTensor& sh, at::IntArrayRef shape, std::string i, double os, Cut c) {
    Tensor out = meta_project_forw(rec, rot, sh, shape, i, os, c);
    return std::make_tuple(out, at::empty({2, out.size(0), out.size(1), out.size(2), out.size(3)}, out.options()));
}
std::tuple<Tensor, Tensor, Tensor> meta_project_2d_back_saved(const Tensor& g, const Tensor&, const Tensor&, const Tensor& rec, const Tensor& rot, const OptTensor& sh,
                                                              std::string, double, Cut, bool need_rec_grad) {
    const bool ns = sh.has_value() && sh->defined() && sh->requires_grad();
    return std::make_tuple(need_rec_grad ? at::empty(rec.sizes(), g.options()) : at::empty({0}, rot.options()),
                           rot.requires_grad() ? at::empty_like(rot) : at::empty({0}, rot.options()), ns ? at::empty_like(*sh) : at::empty({0}, rot.options()));
}
std::tuple<Tensor, Tensor, Tensor> meta_project_back_saved(const Tensor& g, const Tensor&, const Tensor&, const Tensor& rec, const Tensor& rot, const OptTensor& sh,
                                                           std::string, double, Cut, const OptTensor&, bool need_rec_grad) {
    const bool ns = sh.has_value() && sh->defined() && sh->requires_grad();
    return std::make_tuple(need_rec_grad ? at::empty(rec.sizes(), g.options()) : at::empty({0}, rot.options()),
                           rot.requires_grad() ? at::empty_like(rot) : at::empty({0}, rot.options()), ns ? at::empty_like(*sh) : at::empty({0}, rot.options()));
}
Tensor meta_plane_locality_order(const Tensor& rot, int64_t batch) { return at::empty({batch * rot.size(1)}, rot.options().dtype(at::kInt)); }

}  // namespace

// Schema strings verbatim from the reference (csrc/torch_projectors.cpp:23-36).
#define B200PROJ_PROJECT_FORW "(Tensor reconstruction, Tensor rotations, Tensor? shifts, int[] output_shape, str interpolation, float oversampling, float? fourier_radius_cutoff) -> Tensor"
#define B200PROJ_PROJECT_BACK "(Tensor grad_projections, Tensor reconstruction, Tensor rotations, Tensor? shifts, str interpolation, float oversampling, float? fourier_radius_cutoff) -> (Tensor, Tensor, Tensor)"
#define B200PROJ_BACKPROJECT_FORW "(Tensor projections, Tensor? weights, Tensor rotations, Tensor? shifts, str interpolation, float oversampling, float? fourier_radius_cutoff) -> (Tensor, Tensor)"
#define B200PROJ_BACKPROJECT_BACK "(Tensor grad_data_rec, Tensor? grad_weight_rec, Tensor projections, Tensor? weights, Tensor rotations, Tensor? shifts, str interpolation, float oversampling, float? fourier_radius_cutoff) -> (Tensor, Tensor, Tensor, Tensor)"

TORCH_LIBRARY(torch_projectors_b200, m) {
    m.def("project_2d_forw" B200PROJ_PROJECT_FORW);
    m.def("project_2d_back" B200PROJ_PROJECT_BACK);
    m.def("backproject_2d_forw" B200PROJ_BACKPROJECT_FORW);
    m.def("backproject_2d_back" B200PROJ_BACKPROJECT_BACK);
    m.def("project_3d_to_2d_forw" B200PROJ_PROJECT_FORW);
    m.def("project_3d_to_2d_back" B200PROJ_PROJECT_BACK);
    m.def("backproject_2d_to_3d_forw" B200PROJ_BACKPROJECT_FORW);
    m.def("backproject_2d_to_3d_back" B200PROJ_BACKPROJECT_BACK);
    // additions: the volume-reading 3D operators with an explicit processing order of the slices
    m.def("project_3d_to_2d_forw_ordered(Tensor reconstruction, Tensor rotations, Tensor? shifts, int[] output_shape, str interpolation, float oversampling, float? fourier_radius_cutoff, Tensor? pose_order) -> Tensor");
    m.def("project_3d_to_2d_back_ordered(Tensor grad_projections, Tensor reconstruction, Tensor rotations, Tensor? shifts, str interpolation, float oversampling, float? fourier_radius_cutoff, Tensor? pose_order) -> (Tensor, Tensor, Tensor)");
    m.def("backproject_2d_to_3d_back_ordered(Tensor grad_data_rec, Tensor? grad_weight_rec, Tensor projections, Tensor? weights, Tensor rotations, Tensor? shifts, str interpolation, float oversampling, float? fourier_radius_cutoff, Tensor? pose_order) -> (Tensor, Tensor, Tensor, Tensor)");
    m.def("plane_locality_order(Tensor rotations, int batch) -> Tensor");
    // additions: forward projection that also returns the pixels' derivatives with respect to their sample positions
    // [dim, B, P, H, W/2+1], and the backward pass that uses them instead of gathering the volume again
    m.def("project_2d_forw_saving(Tensor reconstruction, Tensor rotations, Tensor? shifts, int[] output_shape, str interpolation, float oversampling, float? fourier_radius_cutoff) -> (Tensor, Tensor)");
    m.def("project_2d_back_saved(Tensor grad_projections, Tensor projections, Tensor derivatives, Tensor reconstruction, Tensor rotations, Tensor? shifts, str interpolation, float oversampling, float? fourier_radius_cutoff, bool need_reconstruction_grad) -> (Tensor, Tensor, Tensor)");
    m.def("project_3d_to_2d_forw_saving(Tensor reconstruction, Tensor rotations, Tensor? shifts, int[] output_shape, str interpolation, float oversampling, float? fourier_radius_cutoff, Tensor? pose_order) -> (Tensor, Tensor)");
    m.def("project_3d_to_2d_back_saved(Tensor grad_projections, Tensor projections, Tensor derivatives, Tensor reconstruction, Tensor rotations, Tensor? shifts, str interpolation, float oversampling, float? fourier_radius_cutoff, Tensor? pose_order, bool need_reconstruction_grad) -> (Tensor, Tensor, Tensor)");
    m.def("_set_pose_order_thresholds(int min_volume_bytes, int min_poses) -> ()", &set_pose_order_thresholds);
    m.def("_get_pose_order_thresholds() -> (int, int)", &get_pose_order_thresholds);
}

TORCH_LIBRARY_IMPL(torch_projectors_b200, CUDA, m) {
    m.impl("project_2d_forw", &project_2d_forw);
    m.impl("project_2d_back", &project_2d_back);
    m.impl("backproject_2d_forw", &backproject_2d_forw);
    m.impl("backproject_2d_back", &backproject_2d_back);
    m.impl("project_3d_to_2d_forw", &project_3d_to_2d_forw);
    m.impl("project_3d_to_2d_back", &project_3d_to_2d_back);
    m.impl("backproject_2d_to_3d_forw", &backproject_2d_to_3d_forw);
    m.impl("backproject_2d_to_3d_back", &backproject_2d_to_3d_back);
    m.impl("project_3d_to_2d_forw_ordered", &project_3d_to_2d_forw_ordered);
    m.impl("project_3d_to_2d_back_ordered", &project_3d_to_2d_back_ordered);
    m.impl("backproject_2d_to_3d_back_ordered", &backproject_2d_to_3d_back_ordered);
    m.impl("plane_locality_order", &plane_locality_order);
    m.impl("project_2d_forw_saving", &project_2d_forw_saving);
    m.impl("project_2d_back_saved", &project_2d_back_saved);
    m.impl("project_3d_to_2d_forw_saving", &project_3d_to_2d_forw_saving);
    m.impl("project_3d_to_2d_back_saved", &project_3d_to_2d_back_saved);
}

TORCH_LIBRARY_IMPL(torch_projectors_b200, Meta, m) {
    m.impl("project_2d_forw", &meta_project_forw);
    m.impl("project_3d_to_2d_forw", &meta_project_forw);
    m.impl("project_3d_to_2d_forw_ordered", &meta_project_forw_ordered);
    m.impl("project_2d_back", &meta_project_back);
    m.impl("project_3d_to_2d_back", &meta_project_back);
    m.impl("project_3d_to_2d_back_ordered", &meta_project_back_ordered);
    m.impl("backproject_2d_forw", &meta_backproject_forw<2>);
    m.impl("backproject_2d_to_3d_forw", &meta_backproject_forw<3>);
    m.impl("backproject_2d_back", &meta_backproject_back);
    m.impl("backproject_2d_to_3d_back", &meta_backproject_back);
    m.impl("backproject_2d_to_3d_back_ordered", &meta_backproject_back_ordered);
    m.impl("plane_locality_order", &meta_plane_locality_order);
    m.impl("project_2d_forw_saving", &meta_project_2d_forw_saving);
    m.impl("project_2d_back_saved", &meta_project_2d_back_saved);
    m.impl("project_3d_to_2d_forw_saving", &meta_project_forw_saving);
    m.impl("project_3d_to_2d_back_saved", &meta_project_back_saved);
}
