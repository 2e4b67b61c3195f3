// Python bindings for the reference's custom-op interface (customops.cu) and its native profiler shim
// (pytorch_xpu_extensions/pcl.xpu.profiler/csrc/profiler/profile.dp.cpp:8-69): mark_event / async_memcpy return an
// EventWrapper with get_submit_time / get_start_time / get_end_time / get_elapsed_time (nanoseconds) and wait.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <chrono>
#include <memory>
#include <mutex>

#include "olb_api.h"

namespace {

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
inline void check(int rc, const char* what) { TORCH_CHECK(rc == 0, what, " failed with code ", rc); }

inline bool is_f32(const at::Tensor& t) {
  TORCH_CHECK(t.is_cuda() && (t.scalar_type() == at::kFloat || t.scalar_type() == at::kBFloat16) && t.is_contiguous(),
              "contiguous CUDA fp32 or bf16 tensor expected");
  return t.scalar_type() == at::kFloat;
}
inline const int* iptr(const at::Tensor& t) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kInt && t.is_contiguous(), "contiguous CUDA int32 tensor expected");
  return t.data_ptr<int>();
}
inline int* iptr_mut(at::Tensor& t) { return const_cast<int*>(iptr(t)); }

at::Tensor compute_partial_token_counts(const at::Tensor& selected_experts, at::Tensor& partial_token_counts,
                                        at::Tensor& expert_counts_ep, int64_t expert_start_idx, int64_t expert_end_idx) {
  c10::cuda::CUDAGuard guard(selected_experts.device());
  check(olb_co_partial_token_counts(iptr(selected_experts), static_cast<int>(selected_experts.size(0)),
                                    static_cast<int>(selected_experts.size(1)), static_cast<int>(expert_start_idx),
                                    static_cast<int>(expert_end_idx - expert_start_idx), iptr_mut(partial_token_counts),
                                    iptr_mut(expert_counts_ep), cur_stream()),
        "compute_partial_token_counts");
  return partial_token_counts;
}

void compute_input_and_output_indices(const at::Tensor& selected_experts, const at::Tensor& partial_cum_token_counts,
                                      at::Tensor& input_increment_buffer, const at::Tensor& cum_expert_counts_ep,
                                      at::Tensor& selected_experts_indices, at::Tensor& input_indices,
                                      at::Tensor& output_indices, int64_t expert_start_idx, int64_t expert_end_idx) {
  c10::cuda::CUDAGuard guard(selected_experts.device());
  const int T = static_cast<int>(selected_experts.size(0));
  const int E_loc = static_cast<int>(expert_end_idx - expert_start_idx);
  TORCH_CHECK(input_increment_buffer.numel() >= static_cast<int64_t>(E_loc) * ((T + 7) / 8), "input_increment_buffer too small");
  check(olb_co_input_output_indices(iptr(selected_experts), T, static_cast<int>(selected_experts.size(1)),
                                    static_cast<int>(expert_start_idx), E_loc, iptr(partial_cum_token_counts),
                                    iptr_mut(input_increment_buffer), iptr(cum_expert_counts_ep),
                                    iptr_mut(selected_experts_indices), iptr_mut(input_indices), iptr_mut(output_indices),
                                    cur_stream()),
        "compute_input_and_output_indices");
}

at::Tensor index_gather(const at::Tensor& inp, const at::Tensor& indices, at::Tensor& out) {
  c10::cuda::CUDAGuard guard(inp.device());
  const bool f32 = is_f32(inp);
  TORCH_CHECK(out.scalar_type() == inp.scalar_type() && out.is_contiguous() && out.size(1) == inp.size(1));
  check(olb_co_index_gather(inp.data_ptr(), iptr(indices), out.data_ptr(), static_cast<int>(indices.numel()),
                            static_cast<int>(inp.size(1)), f32, cur_stream()),
        "index_gather");
  return out;
}

at::Tensor shuffle_sub_matrix_reduce(const at::Tensor& ggemm_input_grad, const at::Tensor& cum_expert_counts_ep,
                                     const at::Tensor& output_indices, at::Tensor& hidden_states_grad) {
  c10::cuda::CUDAGuard guard(ggemm_input_grad.device());
  const bool f32 = is_f32(ggemm_input_grad);
  TORCH_CHECK(hidden_states_grad.scalar_type() == ggemm_input_grad.scalar_type() && hidden_states_grad.is_contiguous());
  check(olb_co_reduce(ggemm_input_grad.data_ptr(), nullptr, 0, iptr(cum_expert_counts_ep), nullptr, iptr(output_indices),
                      hidden_states_grad.data_ptr(), static_cast<int>(hidden_states_grad.size(0)),
                      static_cast<int>(hidden_states_grad.size(1)), 0, f32, cur_stream()),
        "shuffle_sub_matrix_reduce");
  return hidden_states_grad;
}

at::Tensor reduce_ggemm_output(const at::Tensor& ggemm_output, const at::Tensor& routing_weights,
                               const at::Tensor& cum_expert_counts_ep, const at::Tensor& selected_experts_indices,
                               const at::Tensor& output_indices, at::Tensor& final_hidden_states, bool accumulate) {
  c10::cuda::CUDAGuard guard(ggemm_output.device());
  const bool f32 = is_f32(ggemm_output);
  TORCH_CHECK(routing_weights.scalar_type() == ggemm_output.scalar_type() && routing_weights.is_contiguous() &&
              final_hidden_states.scalar_type() == ggemm_output.scalar_type() && final_hidden_states.is_contiguous());
  check(olb_co_reduce(ggemm_output.data_ptr(), routing_weights.data_ptr(), static_cast<int>(routing_weights.size(1)),
                      iptr(cum_expert_counts_ep), iptr(selected_experts_indices), iptr(output_indices),
                      final_hidden_states.data_ptr(), static_cast<int>(final_hidden_states.size(0)),
                      static_cast<int>(final_hidden_states.size(1)), accumulate, f32, cur_stream()),
        "reduce_ggemm_output");
  return final_hidden_states;
}

void reduce_ggemm_output_backward(const at::Tensor& final_hidden_states_grad, const at::Tensor& ggemm_output,
                                  const at::Tensor& routing_weights, const at::Tensor& cum_expert_counts_ep,
                                  const at::Tensor& selected_experts_indices, const at::Tensor& input_indices,
                                  const at::Tensor& output_indices, at::Tensor& ggemm_output_grad,
                                  at::Tensor& routing_weights_grad) {
  (void)input_indices;
  c10::cuda::CUDAGuard guard(ggemm_output.device());
  const bool f32 = is_f32(ggemm_output);
  TORCH_CHECK(final_hidden_states_grad.scalar_type() == ggemm_output.scalar_type() && final_hidden_states_grad.is_contiguous() &&
              routing_weights.scalar_type() == ggemm_output.scalar_type() && routing_weights.is_contiguous() &&
              ggemm_output_grad.scalar_type() == ggemm_output.scalar_type() && ggemm_output_grad.is_contiguous() &&
              routing_weights_grad.scalar_type() == ggemm_output.scalar_type() && routing_weights_grad.is_contiguous());
  check(olb_co_reduce_bwd(final_hidden_states_grad.data_ptr(), ggemm_output.data_ptr(), routing_weights.data_ptr(),
                          static_cast<int>(routing_weights.size(1)), iptr(cum_expert_counts_ep),
                          iptr(selected_experts_indices), iptr(output_indices), ggemm_output_grad.data_ptr(),
                          routing_weights_grad.data_ptr(), static_cast<int>(final_hidden_states_grad.size(0)),
                          static_cast<int>(final_hidden_states_grad.size(1)), f32, cur_stream()),
        "reduce_ggemm_output_backward");
}

at::Tensor index_add_op(const at::Tensor& expert_output, at::Tensor& final_output, const at::Tensor& indices) {
  c10::cuda::CUDAGuard guard(expert_output.device());
  const bool f32 = is_f32(expert_output);
  TORCH_CHECK(final_output.scalar_type() == expert_output.scalar_type() && final_output.is_contiguous() &&
              final_output.size(1) == expert_output.size(1));
  check(olb_co_index_add(expert_output.data_ptr(), final_output.data_ptr(), iptr(indices),
                         static_cast<int>(expert_output.size(0)), static_cast<int>(expert_output.size(1)), f32, cur_stream()),
        "index_add_op");
  return final_output;
}

// ------------------------------------------------------------------------------------------ profiler shim
// Device times come from %globaltimer stamps written by one-thread kernels into pinned, device-mapped slots at the
// stream positions around the measured work; the submit time is the host clock when the work was enqueued.
class StampPool {
 public:
  static StampPool& get() {
    static StampPool pool;
    return pool;
  }
  unsigned long long* take() {
    std::lock_guard<std::mutex> lock(mu_);
    if (!base_) {
      TORCH_CHECK(cudaHostAlloc(reinterpret_cast<void**>(&base_), kSlots * sizeof(unsigned long long), cudaHostAllocMapped) ==
                      cudaSuccess,
                  "pinned allocation for time stamps failed");
    }
    unsigned long long* p = base_ + next_;
    next_ = (next_ + 2) % kSlots;   // slots are handed out in pairs and reused round-robin
    p[0] = p[1] = 0;
    return p;
  }

 private:
  static constexpr int kSlots = 8192;
  unsigned long long* base_ = nullptr;
  int next_ = 0;
  std::mutex mu_;
};

class EventWrapper {
 public:
  EventWrapper(unsigned long long* stamps, cudaEvent_t done, unsigned long long submit_ns)
      : stamps_(stamps), done_(done, [](cudaEvent_t e) { cudaEventDestroy(e); }), submit_ns_(submit_ns) {}
  unsigned long long get_submit_time() const { return submit_ns_; }
  unsigned long long get_start_time() const { sync(); return stamps_[0]; }
  unsigned long long get_end_time() const { sync(); return stamps_[1]; }
  unsigned long long get_elapsed_time() const { sync(); return stamps_[1] - stamps_[0]; }
  void wait() const { sync(); }

 private:
  void sync() const { TORCH_CHECK(cudaEventSynchronize(done_.get()) == cudaSuccess, "event synchronisation failed"); }
  unsigned long long* stamps_;
  std::shared_ptr<std::remove_pointer<cudaEvent_t>::type> done_;
  unsigned long long submit_ns_;
};

unsigned long long host_now_ns() {
  return static_cast<unsigned long long>(
      std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::system_clock::now().time_since_epoch()).count());
}

EventWrapper finish(unsigned long long* stamps, unsigned long long submit_ns, cudaStream_t stream) {
  check(olb_stamp_globaltimer(stamps + 1, stream), "olb_stamp_globaltimer");
  cudaEvent_t done;
  TORCH_CHECK(cudaEventCreateWithFlags(&done, cudaEventDisableTiming) == cudaSuccess, "event creation failed");
  TORCH_CHECK(cudaEventRecord(done, stream) == cudaSuccess, "event record failed");
  return EventWrapper(stamps, done, submit_ns);
}

// A time stamp at the current position of the current stream (start == end).
EventWrapper mark_event() {
  cudaStream_t stream = cur_stream();
  unsigned long long* stamps = StampPool::get().take();
  const unsigned long long submit = host_now_ns();
  check(olb_stamp_globaltimer(stamps, stream), "olb_stamp_globaltimer");
  return finish(stamps, submit, stream);
}

// dst <- src (same number of bytes) on the current stream, bracketed by time stamps.
EventWrapper async_memcpy(const at::Tensor& src, at::Tensor& dst) {
  TORCH_CHECK(src.is_contiguous() && dst.is_contiguous() && src.numel() * src.element_size() == dst.numel() * dst.element_size(),
              "async_memcpy: contiguous tensors of equal byte size expected");
  cudaStream_t stream = cur_stream();
  unsigned long long* stamps = StampPool::get().take();
  const unsigned long long submit = host_now_ns();
  check(olb_stamp_globaltimer(stamps, stream), "olb_stamp_globaltimer");
  TORCH_CHECK(cudaMemcpyAsync(dst.data_ptr(), src.data_ptr(), src.numel() * src.element_size(), cudaMemcpyDefault, stream) ==
                  cudaSuccess,
              "cudaMemcpyAsync failed");
  return finish(stamps, submit, stream);
}

}  // namespace

void register_customops(pybind11::module& m) {
  namespace py = pybind11;
  m.def("co_compute_partial_token_counts", &compute_partial_token_counts);
  m.def("co_compute_input_and_output_indices", &compute_input_and_output_indices);
  m.def("co_index_gather", &index_gather);
  m.def("co_shuffle_sub_matrix_reduce", &shuffle_sub_matrix_reduce);
  m.def("co_reduce_ggemm_output", &reduce_ggemm_output);
  m.def("co_reduce_ggemm_output_backward", &reduce_ggemm_output_backward);
  m.def("co_index_add_op", &index_add_op);
  py::class_<EventWrapper>(m, "EventWrapper")
      .def("get_submit_time", &EventWrapper::get_submit_time)
      .def("get_start_time", &EventWrapper::get_start_time)
      .def("get_end_time", &EventWrapper::get_end_time)
      .def("get_elapsed_time", &EventWrapper::get_elapsed_time)
      .def("wait", &EventWrapper::wait);
  m.def("mark_event", &mark_event, "Time stamp at the current position of the current stream");
  m.def("async_memcpy", &async_memcpy, "Asynchronous copy bracketed by time stamps");
}
