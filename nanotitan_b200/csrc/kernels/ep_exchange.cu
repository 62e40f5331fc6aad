// Expert-parallel row exchange over NVLink peer memory, issued from inside kernels.
//
//  * ep_dispatch: the forward dispatch of a layer in ONE kernel.  Every rank stores its
//    per-expert assignment counts into row `rank` of every peer's count matrix and raises its
//    entry flag; once all flags are up each rank holds C[s][e] = assignments rank s sends to
//    global expert e, from which every row's final position on its expert's rank follows.  The
//    kernel then reads each token row once and stores it, 16 bytes at a time, straight into the
//    expert-major staging buffer of the (up to k) ranks that own its experts - no packed copy
//    on the home rank, no send/receive buffers, no regrouping pass - and leaves through an exit
//    barrier (all rows have landed).  The grouped GEMMs read that staging buffer in place.
//    (The reference does this with an all_to_all_single of counts, a host read of the split
//    sizes, an all_to_all_single of packed rows and a permutation built in Python loops,
//    src/model/torch_backend.py:58-132.)
//  * ep_push_rows: moves rows that already sit in one of the two layouts to the other one on the
//    peers, for the three other transfers of a layer:
//      direction 0 (combine-backward): my rows are packed by global expert; the rows of expert e
//        go to rank e / E_loc, into that rank's expert-major layout (local expert, then source
//        rank, then source order);
//      direction 1 (return and dispatch-backward): my rows are in that expert-major layout; each
//        goes back to the packed position it came from on its source rank.
//    Both layouts are pure functions of the count matrix, so no per-row metadata travels.
//    The entry barrier is optional: a caller may skip it when an earlier barrier of the same
//    layer already orders the peers' last reads of the destination before this launch.
//  * ep_allgather_counts: the count exchange alone (used by the benchmarks).
// All waits are bounded (xrank.cuh); rows that would not fit the destination are skipped and
// reported through the status word.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <ATen/ATen.h>

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
  const XRank& xr = a.xr;
  const uint32_t epoch = xr_begin(xr);
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  // nobody may still be reading the previous matrix: entry barrier first
  if (!xr_barrier(xr, epoch, 0, true, kKernelEpDispatch)) s_ok = 0;
  __syncthreads();
  if (s_ok) {
    for (int i = threadIdx.x; i < a.E * xr.N; i += blockDim.x) {
      const int peer = i / a.E, e = i - peer * a.E;
      a.cmat_peer[peer][xr.rank * a.E + e] = a.counts[e];
    }
  }
  __threadfence_system();
  __syncthreads();
  if (s_ok) xr_barrier(xr, epoch, 1, true, kKernelEpDispatch);
  __syncthreads();
  if (threadIdx.x == 0) xr_end(xr, epoch);
}

// ----------------------------------------------------------------------------- fused forward dispatch
struct DispatchArgs {
  const uint4* x;         // [T, d] token rows
  const float* gates;     // [T, k]
  const int* idx;         // [T, k] expert of each choice
  const int* slot_of;     // [T, k] packed position of each choice on this rank (expert-major, token order)
  const int* counts;      // [E] this rank's assignments per expert
  const int* offsets;     // [E + 1] exclusive scan of counts
  int* cmat_local;        // [ep, E] symmetric: peers write their rows here
  int* cmat_peer[XR_MAX_RANKS];
  uint4* dst_peer[XR_MAX_RANKS];  // expert-side staging [capacity, d] of every rank
  int* cmat_out;          // [ep, E] private copy for the layer's other transfers
  int* local_offsets;     // [E_loc + 1] rows per local expert on this rank (exclusive scan)
  int* packed_token;      // [A]
  float* packed_gate;     // [A]
  long long tokens;
  int k, ep, E, E_loc, vec_per_row;
  long long capacity_rows;
  uint32_t* block_counter;
  XRank xr;
};

__global__ void __launch_bounds__(EP_THREADS)
ep_dispatch_kernel(const DispatchArgs a) {
  __shared__ int seg_peer[EP_MAX_EXPERTS];
  __shared__ int seg_dst0[EP_MAX_EXPERTS];  // first destination row of (me, expert e), minus offsets[e]
  __shared__ int s_ok;
  __shared__ unsigned s_last;
  const XRank& xr = a.xr;
  const uint32_t epoch = xr_begin(xr);
  const int me = xr.rank;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  // ---- counts to every peer, then the entry barrier (block 0 stores and signals, every block waits).
  // A peer that has raised its flag has also finished every earlier kernel of its stream, so its
  // staging buffer is free to be written.
  if (blockIdx.x == 0) {
    for (int i = threadIdx.x; i < a.E * xr.N; i += blockDim.x) {
      const int peer = i / a.E, e = i - peer * a.E;
      a.cmat_peer[peer][me * a.E + e] = a.counts[e];
    }
    __threadfence_system();
    __syncthreads();
  }
  if (!xr_barrier(xr, epoch, 0, blockIdx.x == 0, kKernelEpDispatch)) s_ok = 0;
  __syncthreads();
  // ---- where my rows of expert e start on its rank: experts before e on that rank (all sources),
  // then sources before me for e itself
  const volatile int* cm = a.cmat_local;
  for (int e = threadIdx.x; e < a.E; e += blockDim.x) {
    const int peer = e / a.E_loc;
    int dst0 = 0;
    for (int e2 = peer * a.E_loc; e2 < e; ++e2)
      for (int s = 0; s < a.ep; ++s) dst0 += cm[s * a.E + e2];
    for (int s = 0; s < me; ++s) dst0 += cm[s * a.E + e];
    seg_peer[e] = peer;
    seg_dst0[e] = dst0 - a.offsets[e];
  }
  if (blockIdx.x == 0 && s_ok) {
    for (int i = threadIdx.x; i < a.ep * a.E; i += blockDim.x) a.cmat_out[i] = cm[i];
    if (threadIdx.x == 0) {
      int run = 0;
      a.local_offsets[0] = 0;
      for (int l = 0; l < a.E_loc; ++l) {
        for (int s = 0; s < a.ep; ++s) run += cm[s * a.E + me * a.E_loc + l];
        // rows past the staging capacity were dropped (and reported) by their senders: the GEMMs
        // must not walk past the buffers either
        a.local_offsets[l + 1] = static_cast<int>(min(static_cast<long long>(run), a.capacity_rows));
      }
    }
  }
  __syncthreads();
  if (s_ok) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int warps = EP_THREADS / 32;
    for (long long t = static_cast<long long>(blockIdx.x) * warps + warp; t < a.tokens; t += static_cast<long long>(gridDim.x) * warps) {
      int my_slot = 0, my_e = -1;
      if (lane < a.k) {
        my_slot = a.slot_of[t * a.k + lane];
        my_e = a.idx[t * a.k + lane];
        if (my_slot < 0 || my_slot >= a.tokens * a.k) {  // a slot outside the packed range: skip the choice and report
          report_status(xr.status, kStatusBounds, kKernelEpDispatch, 200000u + static_cast<uint32_t>(lane));
          my_e = -1;
        } else {
          a.packed_token[my_slot] = static_cast<int>(t);
          a.packed_gate[my_slot] = a.gates[t * a.k + lane];
        }
      }
      const uint4* src = a.x + t * a.vec_per_row;
      for (int j = 0; j < a.k; ++j) {
        const int slot = __shfl_sync(0xffffffffu, my_slot, j);
        const int e = __shfl_sync(0xffffffffu, my_e, j);
        if (e < 0 || e >= a.E) {
          if (lane == 0) report_status(xr.status, kStatusBounds, kKernelEpDispatch, static_cast<uint32_t>(e));
          continue;
        }
        const long long dst_row = static_cast<long long>(seg_dst0[e]) + slot;
        if (dst_row < 0 || dst_row >= a.capacity_rows) {  // more rows than the expert rank's staging holds: skip and report
          if (lane == 0) report_status(xr.status, kStatusBounds, kKernelEpDispatch, 100000u + static_cast<uint32_t>(e));
          continue;
        }
        uint4* d = a.dst_peer[seg_peer[e]] + dst_row * a.vec_per_row;
        for (int c = lane; c < a.vec_per_row; c += 32) d[c] = src[c];
      }
    }
  }
  // ---- exit barrier by the last block to finish: every rank's rows have landed
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned ticket = atomicAdd(a.block_counter, 1u);
    s_last = (ticket == gridDim.x - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (s_last) {
    if (threadIdx.x == 0) *a.block_counter = 0u;
    if (s_ok) xr_barrier(xr, epoch, 1, true, kKernelEpDispatch);
    __syncthreads();
    if (threadIdx.x == 0) xr_end(xr, epoch);
  }
}

// ----------------------------------------------------------------------------- layout-to-layout push
struct PushArgs {
  const uint4* src;
  uint4* dst_peer[XR_MAX_RANKS];
  const int* cmat;  // [ep][E] local
  int ep, E, E_loc, direction, entry_barrier;
  int vec_per_row;  // 16-byte vectors per row
  long long dst_capacity_rows, src_rows;
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
  const XRank& xr = a.xr;
  const uint32_t epoch = xr_begin(xr);
  const int me = xr.rank;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (a.entry_barrier && !xr_barrier(xr, epoch, 0, blockIdx.x == 0, kKernelEpDispatch + a.direction)) s_ok = 0;
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
    const long long rows = min(static_cast<long long>(seg_start[a.E]), a.src_rows);
    // Rows are sorted by destination, and every rank would walk the destinations in the same order: all
    // ranks storing into rank 0 first, then into rank 1, ... - one receiver's links busy at a time.  Each
    // rank therefore starts its walk at the first row bound for rank (me + 1) and wraps around, so at any
    // moment the ranks address different receivers.
    long long rot = 0;
    {
      const int first = (me + 1) % a.ep;
      const int g0 = a.direction == 0 ? first * a.E_loc : first;  // first segment whose destination is `first`
      rot = min(static_cast<long long>(seg_start[g0]), rows);
    }
    for (long long r0 = static_cast<long long>(blockIdx.x) * warps + warp; r0 < rows; r0 += static_cast<long long>(gridDim.x) * warps) {
      long long r = r0 + rot;
      if (r >= rows) r -= rows;
      int lo = 0, hi = a.E;  // last segment with seg_start <= r
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (seg_start[mid] <= r) lo = mid; else hi = mid;
      }
      const long long dst_row = seg_dst0[lo] + (r - seg_start[lo]);
      if (dst_row >= a.dst_capacity_rows) {  // would not fit the peer's staging buffer: skip and report
        if (lane == 0) report_status(xr.status, kStatusBounds, kKernelEpDispatch + a.direction, static_cast<uint32_t>(lo));
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
    if (s_ok) xr_barrier(xr, epoch, 1, true, kKernelEpDispatch + a.direction);
    __syncthreads();
    if (threadIdx.x == 0) xr_end(xr, epoch);
  }
}

XRank make_xrank(at::Tensor& flag_local, const at::Tensor& flag_peers, int64_t rank, int64_t world, at::Tensor& epoch_counter, int64_t word_base, double wait_ms) {
  TORCH_CHECK(world >= 1 && world <= XR_MAX_RANKS && flag_peers.numel() == world && flag_peers.scalar_type() == at::kLong, "bad peer flag table");
  TORCH_CHECK(epoch_counter.is_cuda() && epoch_counter.scalar_type() == at::kInt && epoch_counter.numel() >= 1, "epoch counter: one int32 on the device");
  XRank x{};
  x.flag_local = reinterpret_cast<uint32_t*>(flag_local.data_ptr());
  const auto* fp = flag_peers.data_ptr<int64_t>();
  for (int i = 0; i < world; ++i) x.flag_peer[i] = reinterpret_cast<uint32_t*>(fp[i]);
  x.rank = static_cast<int>(rank);
  x.N = static_cast<int>(world);
  x.epoch_counter = reinterpret_cast<uint32_t*>(epoch_counter.data_ptr());
  x.word_base = static_cast<int>(word_base);
  x.wait_cycles = static_cast<long long>(wait_ms * 1.9e6);
  x.status = device_status_word();
  return x;
}

int clamp_grid(int64_t blocks) { return static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(blocks, 148))); }

}  // namespace

// counts [E] int32 (local) -> row `rank` of every peer's [ep, E] matrix (peer table = int64 CPU tensor of device addresses)
void ep_allgather_counts(const at::Tensor& counts, const at::Tensor& cmat_peers, at::Tensor flag_local, const at::Tensor& flag_peers,
                         int64_t rank, int64_t world, at::Tensor epoch_counter, int64_t word_base, double wait_ms) {
  TORCH_CHECK(counts.is_cuda() && counts.scalar_type() == at::kInt && counts.is_contiguous(), "ep_allgather_counts: int32 counts");
  TORCH_CHECK(counts.numel() <= EP_MAX_EXPERTS && cmat_peers.numel() == world, "ep_allgather_counts: sizes");
  c10::cuda::CUDAGuard guard(counts.device());
  CountArgs a{};
  a.counts = counts.data_ptr<int>();
  a.E = static_cast<int>(counts.numel());
  const auto* cp = cmat_peers.data_ptr<int64_t>();
  for (int i = 0; i < world; ++i) a.cmat_peer[i] = reinterpret_cast<int*>(cp[i]);
  a.xr = make_xrank(flag_local, flag_peers, rank, world, epoch_counter, word_base, wait_ms);
  ep_allgather_counts_kernel<<<1, EP_THREADS, 0, at::cuda::getCurrentCUDAStream()>>>(a);
  NT_KERNEL_CHECK();
}

// Forward dispatch of one layer.  x [T, d] 16-bit rows; gates f32 / idx i32 / slot_of i32 [T, k]; counts [E], offsets [E+1] i32.
// cmat_local [ep, E] i32 is this rank's symmetric count matrix (cmat_peers: every rank's), dst_peers the expert-side staging
// buffers [capacity_rows, d].  -> (cmat_out [ep, E], local_offsets [E_loc + 1], packed_token [A] i32, packed_gate [A] f32).
std::vector<at::Tensor> ep_dispatch(const at::Tensor& x, const at::Tensor& gates, const at::Tensor& idx, const at::Tensor& slot_of,
                                    const at::Tensor& counts, const at::Tensor& offsets, at::Tensor cmat_local,
                                    const at::Tensor& cmat_peers, const at::Tensor& dst_peers, int64_t capacity_rows, int64_t E_loc,
                                    at::Tensor block_counter, at::Tensor flag_local, const at::Tensor& flag_peers, int64_t rank,
                                    int64_t world, at::Tensor epoch_counter, double wait_ms, int64_t blocks) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.is_contiguous() && x.element_size() == 2, "ep_dispatch: contiguous 16-bit token rows");
  TORCH_CHECK(x.size(1) % 8 == 0 && reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0, "ep_dispatch: rows must be multiples of 16 bytes");
  TORCH_CHECK(gates.scalar_type() == at::kFloat && gates.is_contiguous() && idx.scalar_type() == at::kInt && idx.is_contiguous() &&
                  slot_of.scalar_type() == at::kInt && slot_of.is_contiguous() && idx.dim() == 2 && idx.size(0) == x.size(0) &&
                  gates.numel() == idx.numel() && slot_of.numel() == idx.numel(),
              "ep_dispatch: gates f32, idx / slot_of i32, all [T, k] contiguous");
  const int64_t E = counts.numel(), k = idx.size(1);
  TORCH_CHECK(counts.scalar_type() == at::kInt && counts.is_contiguous() && offsets.scalar_type() == at::kInt && offsets.is_contiguous() &&
                  offsets.numel() == E + 1 && E <= EP_MAX_EXPERTS && E == E_loc * world && k <= 32,
              "ep_dispatch: counts [E], offsets [E+1] int32, E = E_loc * world <= ", EP_MAX_EXPERTS, ", k <= 32");
  TORCH_CHECK(cmat_local.scalar_type() == at::kInt && cmat_local.numel() == world * E && cmat_peers.numel() == world && dst_peers.numel() == world,
              "ep_dispatch: count matrix / peer tables");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t A = x.size(0) * k;
  auto iopt = counts.options();
  auto cmat_out = at::empty({world, E}, iopt);
  auto local_offsets = at::empty({E_loc + 1}, iopt);
  auto packed_token = at::empty({A}, iopt);
  auto packed_gate = at::empty({A}, gates.options());
  DispatchArgs a{};
  a.x = reinterpret_cast<const uint4*>(x.data_ptr());
  a.gates = gates.data_ptr<float>();
  a.idx = idx.data_ptr<int>();
  a.slot_of = slot_of.data_ptr<int>();
  a.counts = counts.data_ptr<int>();
  a.offsets = offsets.data_ptr<int>();
  a.cmat_local = cmat_local.data_ptr<int>();
  const auto* cp = cmat_peers.data_ptr<int64_t>();
  const auto* dp = dst_peers.data_ptr<int64_t>();
  for (int i = 0; i < world; ++i) {
    a.cmat_peer[i] = reinterpret_cast<int*>(cp[i]);
    a.dst_peer[i] = reinterpret_cast<uint4*>(dp[i]);
  }
  a.cmat_out = cmat_out.data_ptr<int>();
  a.local_offsets = local_offsets.data_ptr<int>();
  a.packed_token = packed_token.data_ptr<int>();
  a.packed_gate = packed_gate.data_ptr<float>();
  a.tokens = x.size(0);
  a.k = static_cast<int>(k);
  a.ep = static_cast<int>(world);
  a.E = static_cast<int>(E);
  a.E_loc = static_cast<int>(E_loc);
  a.vec_per_row = static_cast<int>(x.size(1) / 8);
  a.capacity_rows = capacity_rows;
  a.block_counter = reinterpret_cast<uint32_t*>(block_counter.data_ptr());
  a.xr = make_xrank(flag_local, flag_peers, rank, world, epoch_counter, 0, wait_ms);
  ep_dispatch_kernel<<<clamp_grid(blocks), EP_THREADS, 0, at::cuda::getCurrentCUDAStream()>>>(a);
  NT_KERNEL_CHECK();
  return {cmat_out, local_offsets, packed_token, packed_gate};
}

// src [rows, d] (16-bit) -> peers' staging buffers; see the file comment for the two directions.
void ep_push_rows(const at::Tensor& src, const at::Tensor& dst_peers, int64_t dst_capacity_rows, const at::Tensor& cmat, int64_t E_loc,
                  int64_t direction, bool entry_barrier, at::Tensor block_counter, at::Tensor flag_local, const at::Tensor& flag_peers,
                  int64_t rank, int64_t world, at::Tensor epoch_counter, int64_t word_base, double wait_ms, int64_t blocks) {
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
  a.entry_barrier = entry_barrier ? 1 : 0;
  a.vec_per_row = static_cast<int>(src.size(1) / 8);
  a.dst_capacity_rows = dst_capacity_rows;
  a.src_rows = src.size(0);
  a.block_counter = reinterpret_cast<uint32_t*>(block_counter.data_ptr());
  a.xr = make_xrank(flag_local, flag_peers, rank, world, epoch_counter, word_base, wait_ms);
  ep_push_rows_kernel<<<clamp_grid(blocks), EP_THREADS, 0, at::cuda::getCurrentCUDAStream()>>>(a);
  NT_KERNEL_CHECK();
}

}  // namespace nt
