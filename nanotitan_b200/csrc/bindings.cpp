// Python module `nanotitan_cuda`: the fourteen entry points of the reference's extension
// (csrc/bindings.cpp:59-92 there, same names, argument orders and return conventions) plus
// the kernels the framework itself calls.
#include <torch/extension.h>

#include "cuda_check.h"
#include "kernels/ops.h"
#include "token_loader.h"

namespace py = pybind11;

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "nanotitan_b200 sm_100a kernels";
  // ---- reference-compatible surface
  m.def("random_op", &nt::random_op, "Zero vector of length x with t's options");
  m.def("copy_scalar", &nt::copy_scalar, "Element-wise copy of n elements");
  m.def("copy_vector", &nt::copy_vector, "16-byte vector copy");
  m.def("copy_rows_prefix", &nt::copy_rows_prefix);
  m.def("peer_copy_scalar", &nt::peer_copy_scalar, "GPU-to-GPU copy over NVLink");
  m.def("count_expert_kernel", &nt::count_expert_kernel, "Histogram of expert ids");
  m.def("pack_tokens_kernel", &nt::pack_tokens_kernel, "Pack token rows into expert-major order");
  m.def("combine_tokens_kernel", &nt::combine_tokens_kernel, "Gate-weighted combine of expert rows (fp32 out)");
  m.def("combine_kernel_backward", &nt::combine_kernel_backward, "Backward of combine");
  m.def("gemm_kernel", &nt::gemm_kernel, py::arg("A"), py::arg("B"), py::arg("implementation") = "tiled");
  m.def("tiled_gemm_kernel", &nt::tiled_gemm_kernel);
  m.def("naive_gemm_kernel", &nt::naive_gemm_kernel);
  m.def("pack_kernel_backward", &nt::pack_kernel_backward, "Backward of pack");
  m.def("grouped_gemm_kernel", &nt::grouped_gemm_kernel, "out[r] = X[r] . W[e(r)]");
  m.def("bwd_grouped_gemm_dW_kernel", &nt::bwd_grouped_gemm_dW_kernel);
  m.def("bwd_grouped_gemm_dX_kernel", &nt::bwd_grouped_gemm_dX_kernel);
  // ---- framework kernels
  m.def("gemm_tc", &nt::gemm_tc, py::arg("A"), py::arg("a_mn"), py::arg("Bs"), py::arg("b_mn"), py::arg("b_split"),
        py::arg("Cs"), py::arg("mode") = 0, py::arg("offsets") = py::none(), py::arg("epilogue") = 0,
        py::arg("accumulate") = false, py::arg("aux") = py::none(), py::arg("aux_out") = py::none(),
        py::arg("force_bn") = 0);
  m.def("flash_fwd", &nt::flash_fwd, "Causal flash attention forward -> (out, lse)");
  m.def("flash_bwd", &nt::flash_bwd, py::arg("dout"), py::arg("q"), py::arg("k"), py::arg("v"), py::arg("out"), py::arg("lse"),
        py::arg("scale"), py::arg("grads") = std::vector<at::Tensor>{}, "Causal flash attention backward -> (dq, dk, dv)");
  m.def("bucket_allreduce", &nt::bucket_allreduce, "Fused bucket all-reduce (+ AdamW) over peer / multicast memory");
  m.def("ep_allgather_counts", &nt::ep_allgather_counts, "All-gather per-expert counts through peer stores");
  m.def("ep_dispatch", &nt::ep_dispatch, "Fused count exchange + pack + push of token rows into the expert ranks' staging buffers");
  m.def("ep_push_rows", &nt::ep_push_rows, "Push rows into peers' staging buffers (expert-parallel dispatch / return)");
  m.def("layer_norm_fwd", &nt::layer_norm_fwd);
  m.def("layer_norm_bwd", &nt::layer_norm_bwd, py::arg("dy"), py::arg("x"), py::arg("gamma"), py::arg("mean"), py::arg("rstd"),
        py::arg("dres") = py::none(), py::arg("dgamma_out") = py::none(), py::arg("dbeta_out") = py::none());
  m.def("cross_entropy_fwd_bwd", &nt::cross_entropy_fwd_bwd);
  m.def("adamw_step", &nt::adamw_step, py::arg("param"), py::arg("grad"), py::arg("master"), py::arg("m"), py::arg("v"), py::arg("step"),
        py::arg("lr"), py::arg("beta1"), py::arg("beta2"), py::arg("eps"), py::arg("wd"), py::arg("grad_scale"), py::arg("want_sq"),
        py::arg("bc_dev") = py::none());
  m.def("router_topk", &nt::router_topk);
  m.def("router_from_logits", &nt::router_from_logits, "router_topk's outputs from fp32 logits [T, E]");
  m.def("router_bwd", &nt::router_bwd);
  m.def("assign_slots", &nt::assign_slots);
  m.def("pack_fwd", &nt::pack_fwd);
  m.def("combine_fwd", &nt::combine_fwd);
  m.def("combine_bwd", &nt::combine_bwd);
  m.def("pack_bwd", &nt::pack_bwd);
  m.def("symm_heap_open", &nt::symm_heap_open, py::arg("job"), py::arg("rank"), py::arg("world"), py::arg("device"),
        py::arg("timeout_ms"), "Open this rank's end of a symmetric heap (collective over the ranks of one machine)");
  m.def("symm_heap_alloc", &nt::symm_heap_alloc, py::arg("heap"), py::arg("bytes"), py::arg("multicast"),
        "Collective allocation -> (byte tensor over this rank's piece, every rank's address, multicast address, id)");
  m.def("symm_heap_free", &nt::symm_heap_free);
  m.def("symm_heap_close", &nt::symm_heap_close);
  py::class_<nt::TokenWindowLoader>(m, "TokenWindowLoader",
                                    "Background threads cutting training windows from a uint16 token file into a ring of int64 batches")
      .def(py::init<const std::string&, int64_t, int64_t, int, int>(), py::arg("path"), py::arg("seq_len"), py::arg("batch"),
           py::arg("depth"), py::arg("threads"))
      .def_property_readonly("num_sequences", &nt::TokenWindowLoader::num_sequences)
      .def_property_readonly("slot_elements", &nt::TokenWindowLoader::slot_elements)
      .def_property_readonly("batches_in_epoch", &nt::TokenWindowLoader::batches_in_epoch)
      .def("set_ring",
           [](nt::TokenWindowLoader& self, const at::Tensor& ring, int64_t depth) {
             TORCH_CHECK(ring.device().is_cpu() && ring.scalar_type() == at::kLong && ring.is_contiguous() &&
                             ring.numel() == depth * self.slot_elements(),
                         "ring must be a contiguous int64 host tensor of depth * slot_elements values");
             self.set_ring(ring.data_ptr<int64_t>());
           },
           "The caller keeps `ring` alive while the loader is in use")
      .def("start",
           [](nt::TokenWindowLoader& self, const at::Tensor& order) {
             TORCH_CHECK(order.device().is_cpu() && order.scalar_type() == at::kLong && order.is_contiguous() && order.dim() == 1,
                         "order must be a contiguous 1-D int64 host tensor");
             self.start(order.data_ptr<int64_t>(), order.numel());
           })
      .def("next", &nt::TokenWindowLoader::next, py::arg("timeout_ms"), py::call_guard<py::gil_scoped_release>())
      .def("release", &nt::TokenWindowLoader::release)
      .def("stop", &nt::TokenWindowLoader::stop, py::call_guard<py::gil_scoped_release>());
  m.def("bounded_wait_probe", &nt::bounded_wait_probe, "Let a bounded device wait run out; returns the number of threads that gave up");
  m.def("read_status", &nt::read_status, py::arg("clear") = true, "[code, kernel, detail, count] of the device status word");
  m.def("status_word_tensor", &nt::status_word_tensor);
  m.def("launch_count", [] { return static_cast<long long>(nt::launch_counter().load()); },
        "Kernels of this library launched by this process");
  m.def("launch_counts", [] { return nt::launch_sites().snapshot(); },
        "Kernel launches of this process by host entry point");
}
