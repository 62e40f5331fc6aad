// Tests of the C++ runtime layer (csrc/runtime): RAII stream / event / buffer, the strided view,
// TMA descriptor validation and the device status word.  Plain asserting main(), no framework:
//   nvcc -std=c++17 -gencode arch=compute_100a,code=sm_100a -I nanotitan_b200/csrc/runtime tests/cpp/test_runtime.cu -o test_runtime
#include <cstdio>
#include <stdexcept>
#include <utility>
#include <vector>

#include "cuda_check.h"
#include "cuda_event.h"
#include "cuda_stream.h"
#include "device_buffer.h"
#include "status.h"
#include "tensor_view.h"
#include "tma_desc.h"

static int failures = 0;
#define EXPECT(cond)                                                          \
  do {                                                                        \
    if (!(cond)) { std::printf("FAIL %s:%d  %s\n", __FILE__, __LINE__, #cond); ++failures; } \
  } while (0)

__global__ void fill_view(nt::Tensor2D<float> v, float base) {
  const int i = blockIdx.x, j = threadIdx.x;
  if (v.in_bounds(i, j)) v(i, j) = base + i * 100 + j;
}
__global__ void raise_status(nt::StatusWord* sw) { nt::report_status(sw, nt::kStatusBounds, nt::kKernelProbe, 42u + threadIdx.x); }

static void test_device_buffer_moves() {
  nt::DeviceBuffer<float> a(128);
  float* raw = a.data();
  EXPECT(a.size() == 128 && a.bytes() == 512 && raw != nullptr);
  nt::DeviceBuffer<float> b(std::move(a));
  EXPECT(b.data() == raw && b.size() == 128 && a.data() == nullptr && a.size() == 0);
  nt::DeviceBuffer<float> c;
  c = std::move(b);
  EXPECT(c.data() == raw && b.data() == nullptr);
  nt::DeviceBuffer<float> empty(0);
  EXPECT(empty.data() == nullptr && empty.bytes() == 0);
}

static void test_stream_event_and_view() {
  nt::CudaStream s1, s2;
  nt::CudaStream moved(std::move(s2));
  EXPECT(moved.get() != nullptr && s2.get() == nullptr);
  nt::DeviceBuffer<float> buf(6 * 8);
  buf.zero(s1.get());
  nt::Tensor2D<float> view(buf.data(), 6, 5, 8);  // 5 of 8 columns: padded rows
  nt::CudaEvent start, stop;
  start.record(s1.get());
  fill_view<<<6, 8, 0, s1.get()>>>(view, 1.f);
  NT_KERNEL_CHECK();
  stop.record(s1.get());
  stop.wait(moved.get());  // other stream waits on the device
  moved.synchronize();
  EXPECT(stop.elapsed_ms_since(start) >= 0.f);
  std::vector<float> host(48);
  NT_CUDA_CHECK(cudaMemcpy(host.data(), buf.data(), buf.bytes(), cudaMemcpyDeviceToHost));
  EXPECT(host[0] == 1.f && host[8 + 4] == 105.f && host[5] == 0.f);  // column 5 is outside the view
  nt::CudaEvent e2(std::move(stop));
  EXPECT(e2.get() != nullptr && stop.get() == nullptr);
  EXPECT(nt::launch_counter().load() >= 1);
}

static void test_cuda_check_throws() {
  bool threw = false;
  try {
    NT_CUDA_CHECK(cudaSetDevice(9999));
  } catch (const std::runtime_error& e) {
    threw = std::string(e.what()).find("test_runtime.cu") != std::string::npos;
  }
  cudaGetLastError();
  EXPECT(threw);
}

static void test_tma_descriptor_rules() {
  nt::DeviceBuffer<uint16_t> buf(256 * 512);
  const uint64_t dims[2] = {512, 256};
  const uint64_t strides[1] = {512 * 2};
  const uint32_t box[2] = {64, 128};
  bool ok = true;
  try { (void)nt::make_tma_desc(buf.data(), 2, 2, dims, strides, box, true); } catch (const std::exception&) { ok = false; }
  EXPECT(ok);
  auto rejects = [&](const void* base, const uint64_t* st, const uint32_t* bx) {
    try { (void)nt::make_tma_desc(base, 2, 2, dims, st, bx, true); } catch (const std::runtime_error&) { return true; }
    return false;
  };
  const uint64_t bad_stride[1] = {1022};
  const uint32_t wide_box[2] = {128, 128};
  EXPECT(rejects(buf.data() + 1, strides, box));  // base not 16-byte aligned
  EXPECT(rejects(buf.data(), bad_stride, box));   // stride not a multiple of 16 bytes
  EXPECT(rejects(buf.data(), strides, wide_box)); // inner box wider than the swizzle span
}

static void test_status_word() {
  nt::DeviceBuffer<nt::StatusWord> sw(1);
  sw.zero();
  raise_status<<<1, 32>>>(sw.data());
  NT_KERNEL_CHECK();
  nt::StatusWord host;
  NT_CUDA_CHECK(cudaMemcpy(&host, sw.data(), sizeof(host), cudaMemcpyDeviceToHost));
  EXPECT(host.code == nt::kStatusBounds && host.kernel == nt::kKernelProbe && host.count == 32 && host.detail >= 42 && host.detail < 74);
}

int main() {
  test_device_buffer_moves();
  test_stream_event_and_view();
  test_cuda_check_throws();
  test_tma_descriptor_rules();
  test_status_word();
  std::printf(failures == 0 ? "ALL PASSED\n" : "%d FAILED\n", failures);
  return failures == 0 ? 0 : 1;
}
