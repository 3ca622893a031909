// C++ autograd node of the fused linear: forward Y = X W^T (+ b); backward enqueues dX = dY W and then
// the fused weight-gradient + optimizer update through the C ABI (forge_wgrad_update /
// forge_wgrad_update_group), without entering Python.  It takes the place of the reference's
// FusedLinearAutograd (csrc/fused_linear_cpp/fused_linear.cpp:41-134), which was written to remove the
// per-linear Python overhead of ~225 autograd nodes per step but still calls back into Python (with
// the GIL) for the kernel itself; this node calls the library directly with raw pointers and the
// current CUDA stream.
//
// Only the plain fused branch lives here (an optimizer config is set, no gradient accumulation is
// pending, bf16 activations); the Python autograd function keeps every other branch of the
// reference's table (src/fused_grad_optimizer/autograd.py:61-88).
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include <cstring>
#include <memory>
#include <unordered_set>
#include <vector>

#include "../../include/forge_b200.h"

namespace {

bool g_use_forge_dgrad = false;

void check(int rc, const char* what) {
  TORCH_CHECK(rc == FORGE_OK, what, ": ", forge_last_error_string(), " (code ", rc, ")");
}

// The updates of a fixed set of weights issued as one launch once every member's backward has run.
struct NativeGroup {
  std::unordered_set<const void*> members;
  std::unordered_set<const void*> seen;
  std::vector<ForgeWgradArgs> args;
  std::vector<at::Tensor> keep;   // the recorded activations stay alive until the launch is enqueued
  int device = -1;

  void flush() {
    if (args.empty()) {
      seen.clear();
      return;
    }
    std::vector<ForgeWgradArgs> a;
    a.swap(args);
    std::vector<at::Tensor> k;
    k.swap(keep);
    seen.clear();
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
    check(forge_wgrad_update_group(a.data(), static_cast<int32_t>(a.size()),
                                   c10::cuda::getCurrentCUDAStream(static_cast<c10::DeviceIndex>(device)).stream()),
          "forge_wgrad_update_group");
  }

  void add(const ForgeWgradArgs& a, const at::Tensor& dy, const at::Tensor& x, int dev) {
    if (seen.count(a.W)) flush();   // the same linear twice in one pass: issue what is there first
    device = dev;
    args.push_back(a);
    keep.push_back(dy);
    keep.push_back(x);
    seen.insert(a.W);
    if (seen.size() >= members.size()) flush();
  }
};

// One fused linear: the argument block of its update with everything that does not change between
// steps filled in (W, moments, scales, dtypes, optimizer), the hyper-parameters of the coming step,
// and the per-parameter count of updates.
struct NativeLinear {
  ForgeWgradArgs proto;
  int64_t step = 0;
  std::shared_ptr<NativeGroup> group;

  void set_proto(const std::string& bytes) {
    TORCH_CHECK(bytes.size() == sizeof(ForgeWgradArgs), "argument block of ", bytes.size(), " bytes, expected ",
                sizeof(ForgeWgradArgs));
    std::memcpy(&proto, bytes.data(), sizeof(ForgeWgradArgs));
  }
  void set_hyper(double lr, double beta1, double beta2, double eps, double weight_decay, double momentum, bool nesterov,
                 int64_t hyper_device) {
    proto.hyper.lr = lr;
    proto.hyper.beta1 = beta1;
    proto.hyper.beta2 = beta2;
    proto.hyper.eps = eps;
    proto.hyper.weight_decay = weight_decay;
    proto.hyper.momentum = momentum;
    proto.hyper.nesterov = nesterov ? 1 : 0;
    proto.hyper_device = reinterpret_cast<const void*>(hyper_device);
  }
};

class FusedLinearFn : public torch::autograd::Function<FusedLinearFn> {
 public:
  static at::Tensor forward(torch::autograd::AutogradContext* ctx, const at::Tensor& input, const at::Tensor& weight,
                            const c10::optional<at::Tensor>& bias, int64_t handle) {
    ctx->save_for_backward({input, weight});
    ctx->saved_data["handle"] = handle;
    ctx->saved_data["has_bias"] = bias.has_value() && bias->defined();
    return at::linear(input, weight, bias);
  }

  static torch::autograd::variable_list backward(torch::autograd::AutogradContext* ctx,
                                                 torch::autograd::variable_list grad_outputs) {
    const auto saved = ctx->get_saved_variables();
    const at::Tensor& input = saved[0];
    const at::Tensor& weight = saved[1];
    const at::Tensor& grad_output = grad_outputs[0];
    NativeLinear* h = reinterpret_cast<NativeLinear*>(ctx->saved_data["handle"].toInt());
    const int64_t V = weight.size(0), H = weight.size(1);
    const int dev = weight.get_device();
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(dev));
    cudaStream_t stream = c10::cuda::getCurrentCUDAStream(static_cast<c10::DeviceIndex>(dev)).stream();

    at::Tensor dy2d = grad_output.reshape({-1, V});
    if (!dy2d.is_contiguous()) dy2d = dy2d.contiguous();
    at::Tensor x2d = input.reshape({-1, H});
    if (!x2d.is_contiguous()) x2d = x2d.contiguous();
    const int64_t BT = dy2d.size(0);

    // before any in-place update of `weight` on this stream
    at::Tensor grad_input;
    if (ctx->needs_input_grad(0)) {
      if (g_use_forge_dgrad && weight.scalar_type() == at::kBFloat16 && weight.stride(1) == 1) {
        at::Tensor dx = at::empty({BT, H}, dy2d.options());
        check(forge_dgrad(dy2d.data_ptr(), weight.data_ptr(), dx.data_ptr(), BT, V, H, V, weight.stride(0), H,
                          h->proto.status, stream),
              "forge_dgrad");
        grad_input = dx.reshape(input.sizes());
      } else {
        grad_input = at::matmul(grad_output, weight);
      }
    }

    ForgeWgradArgs a = h->proto;
    a.dY = dy2d.data_ptr();
    a.X = x2d.data_ptr();
    a.BT = BT;
    a.ld_dy = V;
    a.ld_x = H;
    h->step += 1;
    a.hyper.step = static_cast<int32_t>(h->step);
    if (a.state.mode == FORGE_ST_FP8_TENSOR && a.optimizer == FORGE_OPT_ADAMW)
      check(forge_fp8_prestep(a.state.m_scale, a.state.v_scale, a.state.m_absmax_next, a.state.v_absmax_next, stream),
            "forge_fp8_prestep");
    if (h->group) {
      h->group->add(a, dy2d, x2d, dev);
    } else {
      check(forge_wgrad_update(&a, stream), "forge_wgrad_update");
    }
    at::Tensor grad_bias;
    if (ctx->saved_data["has_bias"].toBool()) grad_bias = dy2d.sum(0);
    return {grad_input, at::Tensor(), grad_bias, at::Tensor()};
  }
};

at::Tensor fused_linear(const at::Tensor& input, const at::Tensor& weight, const c10::optional<at::Tensor>& bias,
                        const std::shared_ptr<NativeLinear>& handle) {
  return FusedLinearFn::apply(input, weight, bias, reinterpret_cast<int64_t>(handle.get()));
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "C++ autograd node of forge_b200.FusedLinear";
  pybind11::class_<NativeGroup, std::shared_ptr<NativeGroup>>(m, "Group")
      .def(pybind11::init<>())
      .def("set_members",
           [](NativeGroup& g, const std::vector<int64_t>& ptrs) {
             g.members.clear();
             for (int64_t p : ptrs) g.members.insert(reinterpret_cast<const void*>(p));
           })
      .def("flush", &NativeGroup::flush)
      .def("add_recorded",
           [](NativeGroup& g, const std::string& bytes, int device) {
             // an update recorded by a member whose backward ran in Python; the caller keeps its tensors alive
             TORCH_CHECK(bytes.size() == sizeof(ForgeWgradArgs), "argument block of ", bytes.size(), " bytes, expected ",
                         sizeof(ForgeWgradArgs));
             ForgeWgradArgs a;
             std::memcpy(&a, bytes.data(), sizeof(ForgeWgradArgs));
             g.add(a, at::Tensor(), at::Tensor(), device);
           })
      .def("pending", [](const NativeGroup& g) { return g.args.size(); });
  pybind11::class_<NativeLinear, std::shared_ptr<NativeLinear>>(m, "Linear")
      .def(pybind11::init<>())
      .def("set_proto", [](NativeLinear& h, const pybind11::bytes& b) { h.set_proto(b); })
      .def("set_hyper", &NativeLinear::set_hyper)
      .def("set_group", [](NativeLinear& h, std::shared_ptr<NativeGroup> g) { h.group = std::move(g); })
      .def_readwrite("step", &NativeLinear::step);
  m.def("fused_linear", &fused_linear, "Y = X W^T (+ b); the backward updates W in place through the C ABI");
  m.def("set_use_forge_dgrad", [](bool on) { g_use_forge_dgrad = on; });
  m.def("args_size", []() { return sizeof(ForgeWgradArgs); });
}
