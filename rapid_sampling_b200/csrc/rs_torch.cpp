// PyTorch binding: the three functions of the reference's module (sampling.cpp:5-9) with the same
// names, argument order and tensor semantics, forwarding to the C ABI of this library.
// Argument names follow the reference's README so keyword calls work as well as positional ones.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <map>
#include <mutex>
#include <stdexcept>
#include <string>

#include "../../include/rapid_sampling_b200.h"

namespace {

[[noreturn]] void fail(int rc, const std::string& detail) {
    std::string msg = std::string(rs_status_string(rc)) + detail + " !\n";
    if (rc == RS_ERR_CUDA) throw std::runtime_error(msg + rs_last_cuda_error());
    throw std::invalid_argument(msg);  // pybind11 maps this to ValueError, as in the reference
}

// One zero-initialised workspace per (device, stream); grows, never shrinks, and is kept for the life of the
// process (release_workspaces() drops them).  Returned by value: the reference count is taken under the lock, so a
// concurrent call that grows the same entry cannot free the buffer under a caller that still uses it.  Growing
// allocates: the first call with a given shape must come before any stream capture.
std::mutex g_ws_mu;
std::map<std::pair<int, cudaStream_t>, at::Tensor> g_ws_cache;
at::Tensor workspace_for(int device, cudaStream_t stream, size_t bytes) {
    std::lock_guard<std::mutex> lk(g_ws_mu);
    at::Tensor& w = g_ws_cache[{device, stream}];
    if (!w.defined() || (size_t)w.numel() < bytes)
        w = at::zeros({(int64_t)bytes}, at::TensorOptions().dtype(at::kByte).device(at::kCUDA, device));
    return w;
}

// Host mirror of the device status word, one pinned int per device: the kernels store a non-zero status there as
// well, so a failure (a bounded wait that gave up, a per-row temperature out of range) is noticed by the NEXT call
// on that device from host memory alone -- no copy, no synchronisation on the hot path.
struct Mirror {
    at::Tensor word;   // pinned int32[1]
};
std::mutex g_mirror_mu;
std::map<int, Mirror> g_mirror;
volatile int* mirror_for(int device) {
    std::lock_guard<std::mutex> lk(g_mirror_mu);
    Mirror& m = g_mirror[device];
    if (!m.word.defined()) {
        m.word = at::zeros({1}, at::TensorOptions().dtype(at::kInt)).pin_memory();
        if (rs_set_status_mirror(m.word.data_ptr<int>()) != RS_OK) throw std::runtime_error("rs_set_status_mirror failed !\n");
    }
    return m.word.data_ptr<int>();
}
// Raises what an earlier call on this device left in the mirror, once.
void raise_pending_status(int device, at::Tensor& ws, cudaStream_t stream) {
    volatile int* w = mirror_for(device);
    const int v = *w;
    if (v == 0) return;
    *w = 0;
    rs_clear_status(ws.data_ptr(), stream);
    std::string msg = "an earlier sampling call on cuda:" + std::to_string(device) + " reported: " + rs_status_string(v) + " !\n";
    if (v == RS_ERR_TEMPERATURE) throw std::invalid_argument(msg);
    throw std::runtime_error(msg);
}

struct Shapes {
    int64_t B, T, V;
    float* pen;
    int dtype;
};

// The reference's argument checks (sampling.cu:451-486, :975-1011) plus the ones it leaves out (device, contiguity,
// size of `states`).
Shapes check_arguments(at::Tensor& logits, at::Tensor* penalties, at::Tensor& states, bool any_dtype) {
    const bool lowp = any_dtype && (logits.dtype() == at::kHalf || logits.dtype() == at::kBFloat16);
    if (logits.dtype() != at::kFloat && !lowp)
        throw std::invalid_argument("Logits tensor must be of type float32 (FP32), got " +
                                    std::string(logits.dtype().name()) + " !\n");
    if (!logits.is_cuda() || !states.is_cuda()) throw std::invalid_argument("logits and states must be CUDA tensors !\n");
    if (logits.dim() < 1 || logits.dim() > 3) throw std::invalid_argument("logits must have shape (V,), (B,V) or (B,T,V) !\n");
    if (!logits.is_contiguous() || !states.is_contiguous()) throw std::invalid_argument("logits and states must be contiguous !\n");
    Shapes sh;
    sh.V = logits.size(-1);
    sh.B = (logits.dim() >= 2) ? logits.size(0) : 1;            // sampling.cu:983
    sh.T = (logits.dim() == 3) ? logits.size(1) : 1;            // sampling.cu:984
    sh.pen = nullptr;
    if (penalties) {
        sh.B = (penalties->dim() == 2) ? penalties->size(0) : 1;        // sampling.cu:459
        if (penalties->dtype() != at::kFloat || !penalties->is_cuda() || !penalties->is_contiguous() ||
            penalties->get_device() != logits.get_device())
            throw std::invalid_argument("penalties must be a contiguous float32 CUDA tensor on the logits' device !\n");
        if (penalties->numel() != sh.B * sh.V) throw std::invalid_argument("penalties must have shape (B, V) !\n");
        if (logits.numel() < sh.B * sh.T * sh.V) throw std::invalid_argument("logits hold fewer rows than penalties !\n");
        sh.pen = penalties->data_ptr<float>();
    }
    if (sh.V > 0 && sh.B > 0 && states.numel() * (int64_t)states.element_size() < sh.B * RS_STATE_BYTES)
        throw std::invalid_argument("states tensor is smaller than B rows of setup_rand output !\n");
    if (states.get_device() != logits.get_device()) throw std::invalid_argument("states must live on the logits' device !\n");
    sh.dtype = logits.dtype() == at::kHalf ? RS_DTYPE_F16 : logits.dtype() == at::kBFloat16 ? RS_DTYPE_BF16 : RS_DTYPE_F32;
    return sh;
}

at::Tensor sample_common(at::Tensor& logits, at::Tensor* penalties, at::Tensor& states, double presence,
                         double repetition, double decay, double temperature, int64_t top_k, double top_p,
                         bool any_dtype = false) {
    const Shapes sh = check_arguments(logits, penalties, states, any_dtype);
    const int64_t B = sh.B, T = sh.T, V = sh.V;
    float* pen = sh.pen;

    c10::cuda::CUDAGuard guard(logits.device());
    const int dev = logits.get_device();
    cudaStream_t stream = at::cuda::getCurrentCUDAStream(dev).stream();
    const size_t wsb = rs_workspace_bytes(B, V);
    at::Tensor ws = workspace_for(dev, stream, wsb);
    raise_pending_status(dev, ws, stream);
    at::Tensor out = at::empty({B > 0 ? B : 0}, at::TensorOptions().dtype(at::kInt).device(logits.device()));
    const int dt = sh.dtype;
    const int rc = rs_sample_typed(logits.data_ptr(), dt, B, T, V, pen, states.data_ptr(), out.data_ptr<int32_t>(), temperature,
                                   top_k, top_p, presence, repetition, decay, ws.data_ptr(), (size_t)ws.numel(), stream,
                                   nullptr, nullptr);
    if (rc == RS_ERR_VOCAB) fail(rc, ", got " + std::to_string(V));
    if (rc == RS_ERR_BATCH) fail(rc, ", got B=" + std::to_string(B) + ", T=" + std::to_string(T));
    if (rc == RS_ERR_TEMPERATURE) fail(rc, ", got " + std::to_string(temperature));
    if (rc != RS_OK) fail(rc, "");
    return out;
}

// Per-row temperature / top_k / top_p tensors (B values each, or None for the neutral value in every row).
const void* row_tensor(const c10::optional<at::Tensor>& t, at::ScalarType want, int64_t B, const at::Tensor& logits,
                       const char* name) {
    if (!t.has_value()) return nullptr;
    if (t->scalar_type() != want || !t->is_cuda() || !t->is_contiguous() || t->numel() != B ||
        t->get_device() != logits.get_device())
        throw std::invalid_argument(std::string(name) + " must be a contiguous CUDA tensor of B values (" +
                                    (want == at::kInt ? "int32" : "float32") + ") on the logits' device !\n");
    return t->data_ptr();
}

}  // namespace

// Returns ids (B,) int32, or (ids, probability of the id, kept mass) when return_prob is set.
pybind11::object batch_sampling_rows(at::Tensor& logits, at::Tensor& states, c10::optional<at::Tensor> temperature,
                                     c10::optional<at::Tensor> top_k, c10::optional<at::Tensor> top_p,
                                     c10::optional<at::Tensor> penalties, double presence_penalty,
                                     double repetition_penalty, double penalty_decay, bool return_prob) {
    at::Tensor* pen_t = penalties.has_value() ? &penalties.value() : nullptr;
    const Shapes sh = check_arguments(logits, pen_t, states, true);
    const void* tp = row_tensor(temperature, at::kFloat, sh.B, logits, "temperature");
    const void* kp = row_tensor(top_k, at::kInt, sh.B, logits, "top_k");
    const void* pp = row_tensor(top_p, at::kFloat, sh.B, logits, "top_p");
    c10::cuda::CUDAGuard guard(logits.device());
    const int dev = logits.get_device();
    cudaStream_t stream = at::cuda::getCurrentCUDAStream(dev).stream();
    at::Tensor ws = workspace_for(dev, stream, rs_rows_workspace_bytes(sh.B, sh.V));
    raise_pending_status(dev, ws, stream);
    const int64_t n = sh.B > 0 ? sh.B : 0;
    at::Tensor out = at::empty({n}, at::TensorOptions().dtype(at::kInt).device(logits.device()));
    at::Tensor prob, kept;
    if (return_prob) {
        prob = at::empty({n}, at::TensorOptions().dtype(at::kFloat).device(logits.device()));
        kept = at::empty({n}, at::TensorOptions().dtype(at::kFloat).device(logits.device()));
    }
    const int rc = rs_sample_rows(logits.data_ptr(), sh.dtype, sh.B, sh.T, sh.V, sh.pen, states.data_ptr(), out.data_ptr<int32_t>(),
                                  (const float*)tp, (const int32_t*)kp, (const float*)pp, presence_penalty, repetition_penalty,
                                  penalty_decay, return_prob ? prob.data_ptr<float>() : nullptr,
                                  return_prob ? kept.data_ptr<float>() : nullptr, ws.data_ptr(), (size_t)ws.numel(), stream);
    if (rc == RS_ERR_VOCAB) fail(rc, ", got " + std::to_string(sh.V));
    if (rc == RS_ERR_BATCH) fail(rc, ", got B=" + std::to_string(sh.B) + ", T=" + std::to_string(sh.T));
    if (rc != RS_OK) fail(rc, "");
    if (return_prob) return pybind11::make_tuple(out, prob, kept);
    return pybind11::cast(out);
}

at::Tensor setup_rand(int64_t seed, int64_t B) {
    if (B <= 0) throw std::invalid_argument("B must be positive, got B=" + std::to_string(B) + " !\n");
    at::Tensor state = at::empty({B * RS_STATE_BYTES}, at::TensorOptions().dtype(at::kChar).device(at::kCUDA));
    const int rc = rs_setup_rand(state.data_ptr(), (uint64_t)seed, B, 0, at::cuda::getCurrentCUDAStream().stream());
    if (rc != RS_OK) fail(rc, "");
    return state;
}

at::Tensor batch_sampling_temperature_topk_topp(at::Tensor& logits, at::Tensor& states, double temperature, int64_t top_k,
                                                double top_p) {
    return sample_common(logits, nullptr, states, 0.0, 0.0, 0.0, temperature, top_k, top_p);
}

at::Tensor batch_sampling_repetition_temperature_topk_topp(at::Tensor& logits, at::Tensor& penalties, at::Tensor& states,
                                                           double presence_penalty, double repetition_penalty,
                                                           double penalty_decay, double temperature, int64_t top_k,
                                                           double top_p) {
    return sample_common(logits, &penalties, states, presence_penalty, repetition_penalty, penalty_decay, temperature,
                         top_k, top_p);
}

// The same two calls for fp32, fp16 or bf16 logits (the reference's functions above stay fp32-only, as the reference's).
at::Tensor sample_any(at::Tensor& logits, at::Tensor& states, double temperature, int64_t top_k, double top_p) {
    return sample_common(logits, nullptr, states, 0.0, 0.0, 0.0, temperature, top_k, top_p, true);
}
at::Tensor sample_repetition_any(at::Tensor& logits, at::Tensor& penalties, at::Tensor& states, double presence_penalty,
                                 double repetition_penalty, double penalty_decay, double temperature, int64_t top_k,
                                 double top_p) {
    return sample_common(logits, &penalties, states, presence_penalty, repetition_penalty, penalty_decay, temperature,
                         top_k, top_p, true);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    namespace py = pybind11;
    m.def("setup_rand", &setup_rand, py::arg("seed"), py::arg("B"));
    m.def("batch_sampling_repetition_temperature_topk_topp", &batch_sampling_repetition_temperature_topk_topp,
          py::arg("logits"), py::arg("penalties"), py::arg("states"), py::arg("presence_penalty"),
          py::arg("repetition_penalty"), py::arg("penalty_decay"), py::arg("temperature"), py::arg("top_k"),
          py::arg("top_p"));
    m.def("batch_sampling_temperature_topk_topp", &batch_sampling_temperature_topk_topp, py::arg("logits"),
          py::arg("states"), py::arg("temperature"), py::arg("top_k"), py::arg("top_p"));
    m.def("batch_sampling_temperature_topk_topp_any", &sample_any, py::arg("logits"), py::arg("states"),
          py::arg("temperature"), py::arg("top_k"), py::arg("top_p"));
    m.def("batch_sampling_repetition_temperature_topk_topp_any", &sample_repetition_any, py::arg("logits"),
          py::arg("penalties"), py::arg("states"), py::arg("presence_penalty"), py::arg("repetition_penalty"),
          py::arg("penalty_decay"), py::arg("temperature"), py::arg("top_k"), py::arg("top_p"));
    m.def("batch_sampling_rows", &batch_sampling_rows, py::arg("logits"), py::arg("states"), py::arg("temperature") = py::none(),
          py::arg("top_k") = py::none(), py::arg("top_p") = py::none(), py::arg("penalties") = py::none(),
          py::arg("presence_penalty") = 0.0, py::arg("repetition_penalty") = 0.0, py::arg("penalty_decay") = 0.0,
          py::arg("return_prob") = false);
    m.def("kernel_launch_count", []() { return rs_kernel_launch_count(); });
    m.def("device_status", []() {
        // Synchronises the current stream and returns the status word of its workspace (0 = ok), clearing word and mirror.
        const int dev = c10::cuda::current_device();
        cudaStream_t stream = at::cuda::getCurrentCUDAStream(dev).stream();
        at::Tensor ws = workspace_for(dev, stream, 256);
        int v = rs_device_status(ws.data_ptr(), stream);
        if (v != 0) rs_clear_status(ws.data_ptr(), stream);
        volatile int* w = mirror_for(dev);
        if (v == 0) v = *w;     // a status raised through another workspace of this device
        *w = 0;
        return v;
    });
    m.def("selftest_bounded_wait", [](int64_t polls) {
        // Failure-path instrumentation: one CTA waits on a barrier nothing completes; the next sampling call raises.
        const int dev = c10::cuda::current_device();
        cudaStream_t stream = at::cuda::getCurrentCUDAStream(dev).stream();
        at::Tensor ws = workspace_for(dev, stream, 256);
        mirror_for(dev);
        const int rc = rs_selftest_bounded_wait(ws.data_ptr(), (uint32_t)polls, stream);
        if (rc != RS_OK) fail(rc, "");
    }, py::arg("polls") = 4);
    m.def("release_workspaces", []() {
        std::lock_guard<std::mutex> lk(g_ws_mu);
        g_ws_cache.clear();
    });
    m.def("version", []() { return std::string(rs_version()); });
}
