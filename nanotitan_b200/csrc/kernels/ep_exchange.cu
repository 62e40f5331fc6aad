// Expert-parallel row exchange over NVLink peer memory, issued from inside kernels.
//
//  * ep_allgather_counts: every rank stores its per-expert assignment counts into row `rank` of
//    every peer's count matrix (peer stores) and all ranks meet at a flag barrier, so each rank
//    then holds C[s][e] = assignments rank s sends to global expert e.  (The reference exchanges
//    counts with an all_to_all_single and reads split sizes back to the host,
//    src/model/torch_backend.py:75-96.)
//  * ep_push_rows: moves rows from a local buffer straight to their final position in a peer's
//    staging buffer with 16-byte stores - no send/recv buffers, no regrouping pass:
//      direction 0 (dispatch and combine-backward): my rows are packed by global expert; the rows
//        of expert e go to rank e / E_loc, into that rank's expert-major layout (local expert, then
//        source rank, then source order).
//      direction 1 (return and dispatch-backward): my rows are in that expert-major layout; each
//        goes back to the packed position it came from on its source rank.
//    Both layouts are pure functions of the count matrix, so no per-row metadata travels.
//    The kernel starts with a cross-rank barrier (peers are done with the staging buffer) and ends
//    with one (all rows have landed), see xrank.cuh.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "cuda_check.h"
#include "ops.h"
#include "xrank.cuh"

namespace nt {

namespace {

constexpr int EP_THREADS = 256;
constexpr int EP_MAX_EXPERTS = 256;

struct CountArgs {
  const int* counts;  // [E] local
  int* cmat_peer[XR_MAX_RANKS];
  int E;
  XRank xr;
};

__global__ void __launch_bounds__(EP_THREADS)
ep_allgather_counts_kernel(const CountArgs a) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  // nobody may still be reading the previous matrix: entry barrier first
  if (!xr_barrier(a.xr, 0, true, kKernelEpDispatch)) s_ok = 0;
  __syncthreads();
  if (s_ok) {
    for (int i = threadIdx.x; i < a.E * a.xr.N; i += blockDim.x) {
      const int peer = i / a.E, e = i - peer * a.E;
      a.cmat_peer[peer][a.xr.rank * a.E + e] = a.counts[e];
    }
  }
  __threadfence_system();
  __syncthreads();
  if (s_ok) xr_barrier(a.xr, 1, true, kKernelEpDispatch);
}

struct PushArgs {
  const uint4* src;
  uint4* dst_peer[XR_MAX_RANKS];
  const int* cmat;  // [ep][E] local
  int ep, E, E_loc, direction;
  int vec_per_row;  // 16-byte vectors per row
  long long dst_capacity_rows;
  uint32_t* block_counter;
  XRank xr;
};

__global__ void __launch_bounds__(EP_THREADS)
ep_push_rows_kernel(const PushArgs a) {
  __shared__ int seg_start[EP_MAX_EXPERTS + 1];
  __shared__ int seg_peer[EP_MAX_EXPERTS];
  __shared__ int seg_dst0[EP_MAX_EXPERTS];
  __shared__ int s_ok;
  __shared__ unsigned s_last;
  const int me = a.xr.rank;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (!xr_barrier(a.xr, 0, blockIdx.x == 0, kKernelEpDispatch + a.direction)) s_ok = 0;
  // segment tables (every block builds its own copy; E <= 256 entries)
  for (int g = threadIdx.x; g < a.E; g += blockDim.x) {
    int start = 0, peer, dst0 = 0;
    if (a.direction == 0) {
      const int e = g;
      peer = e / a.E_loc;
      for (int e2 = 0; e2 < e; ++e2) start += a.cmat[me * a.E + e2];
      for (int e2 = peer * a.E_loc; e2 < e; ++e2)
        for (int s = 0; s < a.ep; ++s) dst0 += a.cmat[s * a.E + e2];
      for (int s = 0; s < me; ++s) dst0 += a.cmat[s * a.E + e];
    } else {
      const int e_loc = g / a.ep, s = g - e_loc * a.ep;
      const int e = me * a.E_loc + e_loc;
      peer = s;
      for (int l2 = 0; l2 < e_loc; ++l2)
        for (int s2 = 0; s2 < a.ep; ++s2) start += a.cmat[s2 * a.E + me * a.E_loc + l2];
      for (int s2 = 0; s2 < s; ++s2) start += a.cmat[s2 * a.E + e];
      for (int e2 = 0; e2 < e; ++e2) dst0 += a.cmat[s * a.E + e2];
    }
    seg_start[g] = start;
    seg_peer[g] = peer;
    seg_dst0[g] = dst0;
  }
  if (threadIdx.x == 0) {
    int total = 0;
    if (a.direction == 0) {
      for (int e = 0; e < a.E; ++e) total += a.cmat[me * a.E + e];
    } else {
      for (int l = 0; l < a.E_loc; ++l)
        for (int s = 0; s < a.ep; ++s) total += a.cmat[s * a.E + me * a.E_loc + l];
    }
    seg_start[a.E] = total;
  }
  __syncthreads();
  if (s_ok) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int warps = EP_THREADS / 32;
    const long long rows = seg_start[a.E];
    for (long long r = static_cast<long long>(blockIdx.x) * warps + warp; r < rows; r += static_cast<long long>(gridDim.x) * warps) {
      int lo = 0, hi = a.E;  // last segment with seg_start <= r
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (seg_start[mid] <= r) lo = mid; else hi = mid;
      }
      const long long dst_row = seg_dst0[lo] + (r - seg_start[lo]);
      if (dst_row >= a.dst_capacity_rows) {  // would not fit the peer's staging buffer: skip and report
        if (lane == 0) report_status(a.xr.status, kStatusBounds, kKernelEpDispatch + a.direction, static_cast<uint32_t>(lo));
        continue;
      }
      const uint4* s = a.src + r * a.vec_per_row;
      uint4* d = a.dst_peer[seg_peer[lo]] + dst_row * a.vec_per_row;
      for (int c = lane; c < a.vec_per_row; c += 32) d[c] = s[c];
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned ticket = atomicAdd(a.block_counter, 1u);
    s_last = (ticket == gridDim.x - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (s_last) {
    if (threadIdx.x == 0) *a.block_counter = 0u;
    if (s_ok) xr_barrier(a.xr, 1, true, kKernelEpDispatch + a.direction);
  }
}

XRank make_xrank(at::Tensor& flag_local, const at::Tensor& flag_peers, int64_t rank, int64_t world, int64_t epoch, int64_t word_base, double wait_ms) {
  TORCH_CHECK(world >= 1 && world <= XR_MAX_RANKS && flag_peers.numel() == world && flag_peers.scalar_type() == at::kLong, "bad peer flag table");
  XRank x{};
  x.flag_local = reinterpret_cast<uint32_t*>(flag_local.data_ptr());
  const auto* fp = flag_peers.data_ptr<int64_t>();
  for (int i = 0; i < world; ++i) x.flag_peer[i] = reinterpret_cast<uint32_t*>(fp[i]);
  x.rank = static_cast<int>(rank);
  x.N = static_cast<int>(world);
  x.epoch = static_cast<uint32_t>(epoch);
  x.word_base = static_cast<int>(word_base);
  x.wait_cycles = static_cast<long long>(wait_ms * 1.9e6);
  x.status = device_status_word();
  return x;
}

}  // namespace

// counts [E] int32 (local) -> row `rank` of every peer's [ep, E] matrix (peer table = int64 CPU tensor of device addresses)
void ep_allgather_counts(const at::Tensor& counts, const at::Tensor& cmat_peers, at::Tensor flag_local, const at::Tensor& flag_peers,
                         int64_t rank, int64_t world, int64_t epoch, int64_t word_base, double wait_ms) {
  TORCH_CHECK(counts.is_cuda() && counts.scalar_type() == at::kInt && counts.is_contiguous(), "ep_allgather_counts: int32 counts");
  TORCH_CHECK(counts.numel() <= EP_MAX_EXPERTS && cmat_peers.numel() == world, "ep_allgather_counts: sizes");
  c10::cuda::CUDAGuard guard(counts.device());
  CountArgs a{};
  a.counts = counts.data_ptr<int>();
  a.E = static_cast<int>(counts.numel());
  const auto* cp = cmat_peers.data_ptr<int64_t>();
  for (int i = 0; i < world; ++i) a.cmat_peer[i] = reinterpret_cast<int*>(cp[i]);
  a.xr = make_xrank(flag_local, flag_peers, rank, world, epoch, word_base, wait_ms);
  ep_allgather_counts_kernel<<<1, EP_THREADS, 0, at::cuda::getCurrentCUDAStream()>>>(a);
  NT_KERNEL_CHECK();
}

// src [rows, d] (16-bit) -> peers' staging buffers; see the file comment for the two directions.
void ep_push_rows(const at::Tensor& src, const at::Tensor& dst_peers, int64_t dst_capacity_rows, const at::Tensor& cmat, int64_t E_loc,
                  int64_t direction, at::Tensor block_counter, at::Tensor flag_local, const at::Tensor& flag_peers, int64_t rank,
                  int64_t world, int64_t epoch, int64_t word_base, double wait_ms, int64_t blocks) {
  TORCH_CHECK(src.is_cuda() && src.dim() == 2 && src.is_contiguous() && src.element_size() == 2, "ep_push_rows: contiguous 16-bit rows");
  TORCH_CHECK(src.size(1) % 8 == 0 && reinterpret_cast<uintptr_t>(src.data_ptr()) % 16 == 0, "ep_push_rows: rows must be multiples of 16 bytes");
  TORCH_CHECK(cmat.is_cuda() && cmat.scalar_type() == at::kInt && cmat.is_contiguous() && cmat.dim() == 2 && cmat.size(0) == world, "ep_push_rows: cmat [ep, E] int32");
  TORCH_CHECK(cmat.size(1) <= EP_MAX_EXPERTS && cmat.size(1) == E_loc * world, "ep_push_rows: expert counts");
  c10::cuda::CUDAGuard guard(src.device());
  PushArgs a{};
  a.src = reinterpret_cast<const uint4*>(src.data_ptr());
  const auto* dp = dst_peers.data_ptr<int64_t>();
  for (int i = 0; i < world; ++i) a.dst_peer[i] = reinterpret_cast<uint4*>(dp[i]);
  a.cmat = cmat.data_ptr<int>();
  a.ep = static_cast<int>(world);
  a.E = static_cast<int>(cmat.size(1));
  a.E_loc = static_cast<int>(E_loc);
  a.direction = static_cast<int>(direction);
  a.vec_per_row = static_cast<int>(src.size(1) / 8);
  a.dst_capacity_rows = dst_capacity_rows;
  a.block_counter = reinterpret_cast<uint32_t*>(block_counter.data_ptr());
  a.xr = make_xrank(flag_local, flag_peers, rank, world, epoch, word_base, wait_ms);
  const int grid = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(blocks, 148)));
  ep_push_rows_kernel<<<grid, EP_THREADS, 0, at::cuda::getCurrentCUDAStream()>>>(a);
  NT_KERNEL_CHECK();
}

}  // namespace nt
