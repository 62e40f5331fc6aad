// Causal flash attention for sm_100a: forward, dQ and dK/dV kernels from one template.
//
// All three walk the same dataflow with tcgen05 tensor cores and TMEM accumulators.  A CTA
// keeps a 128-row "resident" tile R in shared memory and streams "column" tiles C past it:
//     T1 = R_a . C_a^T          (128 x BC scores, reduction over the head dim)
//     T2 = R_b . C_b^T          (backward only: dP)
//     E  = f(T1, T2)            (bf16 tile written to shared memory by the 128 softmax threads,
//                                thread i owning row i, so row max / sum need no shuffles)
//     Acc (+)= E . C_x          (128 x Dh, reduction over the BC streamed rows)
//   forward : R = Q_i            C = (K_j, V_j)       E = P           Acc = P V     (rescaled in registers)
//   dQ      : R = (Q_i, dO_i)    C = (K_j, V_j)       E = dS          Acc += dS K
//   dK/dV   : R = (K_j, V_j)     C = (Q_i, dO_i)      E = (P^T, dS^T) Acc += P^T dO, dS^T Q
// The same [rows][Dh] shared-memory tile serves as a K-major operand (reduction over Dh) and as
// an MN-major operand (reduction over rows) through two descriptors.  The S x S score matrix is
// never materialised; the causal mask comes from indices (the reference materialises
// [B, H, S, S] scores and keeps a boolean mask buffer, src/model/model.py:122-176).
// Splitting backward into a dQ pass and a dK/dV pass recomputes the scores once more but needs
// no atomics, so gradients are bit-reproducible.
//
// Warp roles: warp 0 TMA producer, warp 1 MMA issuer (+ TMEM owner), warps 2-9 softmax/epilogue:
// two warpgroups of 128 threads.  Thread i of either warpgroup owns row i of the resident tile
// (a warp reads the TMEM lanes of its quarter, warp % 4), and the two warpgroups split the 64
// streamed columns of a step: warpgroup g works on columns [32 g, 32 g + 32).  In backward the
// halves are independent.  In forward the row maximum is exchanged through shared memory (one
// named barrier per step), each warpgroup keeps its own partial row sum and folds its own half of
// the head dimension of the P.V product; the partial sums meet once, at the end.
// TMEM use is <= 256 columns and shared memory ~100 KB so two CTAs share an SM: 16 softmax warps
// per SM hide the tcgen05.ld and exponential latencies of one another.  Every mbarrier wait is
// bounded (see sm100.cuh); after an abandoned wait a thread keeps walking the loop so that the
// named barriers still see every thread.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <ATen/ATen.h>

#include "cuda_check.h"
#include "ops.h"
#include "sm100.cuh"
#include "tma_desc.h"

#include <cstdlib>
#include <type_traits>

namespace nt {
namespace attn {

enum Mode : int { kFwd = 0, kDq = 1, kDkv = 2 };
constexpr int BR = 128;  // resident rows
constexpr int THREADS = 320;
constexpr int SOFTMAX_THREADS = 256;
constexpr float LOG2E = 1.4426950408889634f;

struct Args {
  int B, H, S;
  float scale;
  int dtype;  // 0 fp16, 1 bf16
  // element strides of the [B, S, H, Dh] outputs (last dim contiguous)
  void* out0;  // fwd: O.  dq: dQ.  dkv: dV
  void* out1;  // dkv: dK
  long long o_sb, o_ss, o_sh;  // batch / seq / head strides (elements) shared by the outputs
  float* lse;        // [B, H, S]  (fwd: written; bwd: read)
  const float* dsum; // [B, H, S]  rowsum(dO * O) (bwd)
  StatusWord* status;
};

template <int DH, int MODE>
struct Cfg {
  static constexpr int BC = 64;                                 // streamed rows per step
  static constexpr int R_TILE = BR * DH * 2;                     // bytes
  static constexpr int C_TILE = BC * DH * 2;
  static constexpr int N_R = MODE == kFwd ? 1 : 2;
  // operand stages of the streamed tiles; dK/dV at head dim 64 keeps two so that two CTAs still fit an SM's shared memory
  static constexpr int STAGES = (MODE == kDkv && DH == 64) ? 2 : 3;
  static constexpr int E_TILE = BR * BC * 2;
  static constexpr int N_E = MODE == kDq ? 1 : 2;                // fwd: P of even / odd steps; dkv: P^T and dS^T
  static constexpr int OFF_R = 0;
  static constexpr int OFF_C = OFF_R + N_R * R_TILE;
  static constexpr int OFF_E = OFF_C + STAGES * 2 * C_TILE;
  static constexpr int OFF_VEC = OFF_E + N_E * E_TILE;           // dkv: lse / dsum of the streamed queries; fwd: row max / sum exchange
  static constexpr int OFF_BAR = OFF_VEC + 4096;
  static constexpr int TOTAL = OFF_BAR + 16 * 8 + 16 + 1024;
  static constexpr uint32_t TMEM_COLS = 256;
  // forward double-buffers T1 (columns 0 and 64); backward keeps T1 at 0 and T2 at 64
  static constexpr uint32_t COL_T1 = 0, COL_T2 = BC, COL_ACC1 = 128, COL_ACC2 = 192;
  static constexpr uint32_t SWZ = DH == 32 ? 4u : 2u;            // 64-byte or 128-byte swizzle for [rows][Dh] tiles
  static constexpr uint32_t ROW_BYTES = DH * 2;
  static constexpr uint32_t SBO_RC = 8 * ROW_BYTES;              // 8-row group pitch of R / C tiles
};

__device__ __forceinline__ uint64_t make_desc(uint32_t addr, uint32_t lbo, uint32_t sbo, uint32_t layout) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;
  d |= static_cast<uint64_t>(layout) << 61;
  return d;
}

__device__ __forceinline__ void named_sync_softmax() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// 32 lanes x 16 consecutive fp32 columns (thread i of the warp receives lane base_lane + i)
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ uint32_t pack_pair(float lo, float hi, int dtype) {
  if (dtype == 1) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Write N (16 or 32) consecutive values of row `r` (columns c0 .. c0+N-1 of a 128 x BC tile) into a K-major,
// 128-byte-swizzled operand tile made of 64-column chunks of [128 rows][128 B].
template <int N>
__device__ __forceinline__ void write_e_chunk(uint8_t* tile, int r, int c0, const float (&v)[N], int dtype) {
  uint8_t* row = tile + (c0 >> 6) * (BR * 128) + r * 128;
  const int u0 = (c0 & 63) >> 3;
#pragma unroll
  for (int u = 0; u < N / 8; ++u) {
    uint4 q;
    q.x = pack_pair(v[8 * u + 0], v[8 * u + 1], dtype);
    q.y = pack_pair(v[8 * u + 2], v[8 * u + 3], dtype);
    q.z = pack_pair(v[8 * u + 4], v[8 * u + 5], dtype);
    q.w = pack_pair(v[8 * u + 6], v[8 * u + 7], dtype);
    *reinterpret_cast<uint4*>(row + (((u0 + u) ^ (r & 7)) << 4)) = q;
  }
}

template <int N>
__device__ __forceinline__ void store_row(void* base, long long off, const float* v, int dtype) {
  uint16_t* p = reinterpret_cast<uint16_t*>(base) + off;
#pragma unroll
  for (int u = 0; u < N / 8; ++u) {
    uint4 q;
    q.x = pack_pair(v[8 * u + 0], v[8 * u + 1], dtype);
    q.y = pack_pair(v[8 * u + 2], v[8 * u + 3], dtype);
    q.z = pack_pair(v[8 * u + 4], v[8 * u + 5], dtype);
    q.w = pack_pair(v[8 * u + 6], v[8 * u + 7], dtype);
    reinterpret_cast<uint4*>(p)[u] = q;
  }
}

// tm0/tm1: resident tensors (box {Dh, 128, 1, 1}); tm2/tm3: streamed tensors (box {Dh, BC, 1, 1}).
// Tensor maps are 4-D over (Dh, H, S, B) so a tile is addressed as (0, h, s0, b).
// DT: 0 = fp16, 1 = bf16 (compile-time so the pack / convert code has no per-element selects)
template <int DH, int MODE, int DT>
__global__ void __launch_bounds__(THREADS, 2)
causal_attn_kernel(const __grid_constant__ CUtensorMap tm0, const __grid_constant__ CUtensorMap tm1,
             const __grid_constant__ CUtensorMap tm2, const __grid_constant__ CUtensorMap tm3, const Args args) {
  using namespace sm100;
  using C = Cfg<DH, MODE>;
  constexpr int BC = C::BC;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint64_t* r_full = bars;            // 1
  uint64_t* c_full = bars + 1;        // STAGES (<= 4)
  uint64_t* c_empty = bars + 5;       // STAGES (<= 4)
  uint64_t* t_full = bars + 9;        // 1 (forward: score buffer 0)
  uint64_t* t_full_b = bars + 10;     // forward: score buffer 1
  uint64_t* e_full = bars + 11;       // 1 (one arrival per softmax warp)
  uint64_t* e_empty = bars + 12;      // 1
  uint64_t* acc_full = bars + 13;     // 1 (forward: accumulator of even steps)
  uint64_t* acc_full_b = bars + 14;   // forward: accumulator of odd steps
  uint64_t* t_empty = bars + 15;      // backward: the softmax warps have read the scores into registers
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rt = gridDim.x - 1 - blockIdx.x;  // heavy (late) tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int r0 = rt * BR;                      // first resident row (query row for fwd/dq, key row for dkv)
  const int S = args.S;

  // streamed tile range [c_begin, c_end)
  int c_begin, c_end;
  if (MODE == kDkv) {
    c_begin = r0 / BC;                                   // queries >= first key of the tile
    c_end = (S + BC - 1) / BC;
  } else {
    c_begin = 0;
    c_end = (min(r0 + BR, S) + BC - 1) / BC;             // keys <= last query of the tile
  }
  // a failure recorded earlier (by any kernel) turns every later CTA into a no-op until the host clears it
  const bool dead = args.status != nullptr && *reinterpret_cast<volatile uint32_t*>(&args.status->code) != 0u;
  const int n_iter = dead ? 0 : c_end - c_begin;

  if (threadIdx.x == 0) {
    mbar_init(r_full, 1);
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(&c_full[s], 1); mbar_init(&c_empty[s], 1); }
    mbar_init(t_full, 1);
    mbar_init(t_full_b, 1);
    mbar_init(e_full, SOFTMAX_THREADS / 32);  // one arrival per softmax warp
    mbar_init(e_empty, 1);
    mbar_init(acc_full, 1);
    mbar_init(acc_full_b, 1);
    mbar_init(t_empty, SOFTMAX_THREADS / 32);
    *abort_flag = 0u;
    fence_barrier_init();
    prefetch_tmap(&tm0);
    prefetch_tmap(&tm2);
    prefetch_tmap(&tm3);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(r_full, C::N_R * C::R_TILE);
      tma_load_4d(smem + C::OFF_R, &tm0, r_full, 0, h, r0, b);
      if (C::N_R == 2) tma_load_4d(smem + C::OFF_R + C::R_TILE, &tm1, r_full, 0, h, r0, b);
      int stage = 0;
      uint32_t phase = 0;
      for (int it = 0; it < n_iter; ++it) {
        if (!mbar_wait(&c_empty[stage], phase ^ 1u, abort_flag, args.status, kKernelAttnFwd + MODE, 100 + stage)) break;
        uint8_t* sc = smem + C::OFF_C + stage * 2 * C::C_TILE;
        mbar_expect_tx(&c_full[stage], 2 * C::C_TILE);
        const int c0 = (c_begin + it) * BC;
        tma_load_4d(sc, &tm2, &c_full[stage], 0, h, c0, b);
        tma_load_4d(sc + C::C_TILE, &tm3, &c_full[stage], 0, h, c0, b);
        if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    const uint32_t idesc_t = umma_idesc(DT, BR, BC, 0, 0);
    const uint32_t idesc_acc = umma_idesc(DT, BR, DH, 0, 1);
    const uint32_t ra = smem_u32(smem + C::OFF_R), rb = ra + C::R_TILE;
    const uint32_t e1 = smem_u32(smem + C::OFF_E), e2 = e1 + C::E_TILE;
    bool ok = mbar_wait(r_full, 0, abort_flag, args.status, kKernelAttnFwd + MODE, 200);
    if (MODE == kFwd) {
      // Forward keeps two score buffers in TMEM: the scores of step it+1 are issued before the
      // softmax threads have finished step it, so they never wait for the tensor core.
      auto issue_scores = [&](int it) -> bool {
        const int st = it % C::STAGES, tb = it & 1;  // operand stage, score buffer
        if (!mbar_wait(&c_full[st], (it / C::STAGES) & 1, abort_flag, args.status, kKernelAttnFwd + MODE, 210 + st)) return false;
        tc_fence_after();
        if (lane == 0) {
          const uint32_t ca = smem_u32(smem + C::OFF_C + st * 2 * C::C_TILE);
#pragma unroll
          for (int ks = 0; ks < DH / 16; ++ks)
            umma_f16(tmem_base + C::COL_T1 + tb * BC, make_desc(ra + ks * 32, 16, C::SBO_RC, C::SWZ),
                     make_desc(ca + ks * 32, 16, C::SBO_RC, C::SWZ), idesc_t, ks != 0);
          umma_commit(tb ? t_full_b : t_full);
        }
        __syncwarp();
        return true;
      };
      if (ok && n_iter > 0) ok = issue_scores(0);
      for (int it = 0; it < n_iter && ok; ++it) {
        if (it + 1 < n_iter && !issue_scores(it + 1)) { ok = false; break; }
        if (!mbar_wait(e_full, it & 1, abort_flag, args.status, kKernelAttnFwd + MODE, 220)) { ok = false; break; }
        tc_fence_after();
        if (lane == 0) {
          const int st = it % C::STAGES;
          const uint32_t cb = smem_u32(smem + C::OFF_C + st * 2 * C::C_TILE) + C::C_TILE;  // V
          const uint32_t ep = (it & 1) ? e2 : e1;
#pragma unroll
          for (int ks = 0; ks < BC / 16; ++ks)
            umma_f16(tmem_base + ((it & 1) ? C::COL_ACC2 : C::COL_ACC1), make_desc(ep + ks * 32, 16, 1024, 2u),
                     make_desc(cb + ks * 2 * C::SBO_RC, 16, C::SBO_RC, C::SWZ), idesc_acc, ks != 0 ? 1u : 0u);
          umma_commit(&c_empty[st]);
          umma_commit((it & 1) ? acc_full_b : acc_full);
        }
        __syncwarp();
      }
    }
    if (MODE != kFwd) {
      // Backward.  T1 / T2 are single-buffered, but the softmax warps release them (t_empty) as soon as
      // the scores sit in their registers, so the score products of step it+1 run under the softmax
      // arithmetic of step it; only the accumulate products wait for the step's E tiles.
      auto issue_t = [&](int it) -> bool {
        const int st = it % C::STAGES;
        if (!mbar_wait(&c_full[st], (it / C::STAGES) & 1, abort_flag, args.status, kKernelAttnFwd + MODE, 210 + st)) return false;
        tc_fence_after();
        if (lane == 0) {
          const uint32_t ca = smem_u32(smem + C::OFF_C + st * 2 * C::C_TILE), cb = ca + C::C_TILE;
#pragma unroll
          for (int ks = 0; ks < DH / 16; ++ks)
            umma_f16(tmem_base + C::COL_T1, make_desc(ra + ks * 32, 16, C::SBO_RC, C::SWZ), make_desc(ca + ks * 32, 16, C::SBO_RC, C::SWZ),
                     idesc_t, ks != 0);
#pragma unroll
          for (int ks = 0; ks < DH / 16; ++ks)
            umma_f16(tmem_base + C::COL_T2, make_desc(rb + ks * 32, 16, C::SBO_RC, C::SWZ), make_desc(cb + ks * 32, 16, C::SBO_RC, C::SWZ),
                     idesc_t, ks != 0);
          umma_commit(t_full);
        }
        __syncwarp();
        return true;
      };
      if (ok && n_iter > 0) ok = issue_t(0);
      for (int it = 0; it < n_iter && ok; ++it) {
        const int st = it % C::STAGES;
        if (it + 1 < n_iter) {
          if (!mbar_wait(t_empty, it & 1, abort_flag, args.status, kKernelAttnFwd + MODE, 215)) { ok = false; break; }
          tc_fence_after();
          if (!issue_t(it + 1)) { ok = false; break; }
        }
        if (!mbar_wait(e_full, it & 1, abort_flag, args.status, kKernelAttnFwd + MODE, 220)) { ok = false; break; }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t ca = smem_u32(smem + C::OFF_C + st * 2 * C::C_TILE), cb = ca + C::C_TILE;
          // Acc (+)= E . C_x with C_x read MN-major: 16 streamed rows per step = two 8-row groups
          const uint32_t cx1 = (MODE == kDq) ? ca : cb;  // dq: K, dkv: dO
          const uint32_t acc_on = it != 0 ? 1u : 0u;
#pragma unroll
          for (int ks = 0; ks < BC / 16; ++ks) {
            const uint32_t e_off = (ks >> 2) * (BR * 128) + (ks & 3) * 32;
            umma_f16(tmem_base + C::COL_ACC1, make_desc(e1 + e_off, 16, 1024, 2u),
                     make_desc(cx1 + ks * 2 * C::SBO_RC, 16, C::SBO_RC, C::SWZ), idesc_acc, (ks != 0) ? 1u : acc_on);
          }
          if (MODE == kDkv) {
#pragma unroll
            for (int ks = 0; ks < BC / 16; ++ks) {
              const uint32_t e_off = (ks >> 2) * (BR * 128) + (ks & 3) * 32;
              umma_f16(tmem_base + C::COL_ACC2, make_desc(e2 + e_off, 16, 1024, 2u),
                       make_desc(ca + ks * 2 * C::SBO_RC, 16, C::SBO_RC, C::SWZ), idesc_acc, (ks != 0) ? 1u : acc_on);
            }
          }
          umma_commit(&c_empty[st]);
          umma_commit(e_empty);
          if (it == n_iter - 1) umma_commit(acc_full);
        }
        __syncwarp();
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax / epilogue (2 x 128 threads)
    const int quarter = warp & 3;           // TMEM lane quarter this warp may read
    const int wg = (warp - 2) >> 2;         // warpgroup: which 32 of the 64 streamed columns
    const int r = quarter * 32 + lane;      // row of the resident tile owned by this thread
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const int row_idx = r0 + r;             // query index (fwd/dq) or key index (dkv)
    const float sl2 = args.scale * LOG2E;
    uint8_t* e1 = smem + C::OFF_E;
    uint8_t* e2 = e1 + C::E_TILE;
    float* vec = reinterpret_cast<float*>(smem + C::OFF_VEC);
    const long long bh = static_cast<long long>(b) * args.H + h;
    constexpr int HD = DH / 2;              // head-dim columns each warpgroup folds / stores
    const int col_half = wg * HD;

    float m_run = -INFINITY, l_run = 0.f;
    float o_acc[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) o_acc[i] = 0.f;
    float my_lse = 0.f, my_dsum = 0.f;
    if (MODE == kDq && row_idx < S) {
      my_lse = args.lse[bh * S + row_idx] * LOG2E;
      my_dsum = args.dsum[bh * S + row_idx];
    }
    bool ok = true;
    if (MODE == kFwd) {
      // The P.V product of step j lands in accumulator j & 1 and is folded into o_acc during step
      // j + 2, so neither its latency nor the hand-offs around it sit on a step's critical path.
      // alpha_j = exp(m_{j-1} - m_j) rescales what was folded before j; a1 / a2 hold it for the two
      // steps whose products are still outstanding.
      float a1 = 0.f, a2 = 0.f;
      float* mx = vec;  // [2 (step parity)][2 (warpgroup)][128]: the warpgroups' row maxima of a step
      // fold this warpgroup's half of the P.V product of step `j` (scaled to that step's row max)
      auto fold_pv = [&](int j, float alpha_j) -> bool {
        if (!mbar_wait((j & 1) ? acc_full_b : acc_full, (j >> 1) & 1, abort_flag, args.status, kKernelAttnFwd + MODE, 320)) return false;
        tc_fence_after();
#pragma unroll
        for (int cc = 0; cc < HD; cc += 16) {
          uint32_t t[16];
          tmem_ld_32x16(lane_addr + ((j & 1) ? C::COL_ACC2 : C::COL_ACC1) + col_half + cc, t);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) o_acc[cc + i] = o_acc[cc + i] * alpha_j + __uint_as_float(t[i]);
        }
        tc_fence_before();
        return true;
      };
      for (int it = 0; it < n_iter; ++it) {  // runs to the end even after an abandoned wait: the named barrier needs every thread
        const int c0 = it * BC + wg * 32;  // first key of this warpgroup's half
        bool step_ok = ok;
        if (step_ok) step_ok = mbar_wait((it & 1) ? t_full_b : t_full, (it >> 1) & 1, abort_flag, args.status, kKernelAttnFwd + MODE, 300);
        uint32_t t[32];
        float m_loc = -INFINITY;
        if (step_ok) {
          tc_fence_after();
          tmem_ld_32x32(lane_addr + C::COL_T1 + (it & 1) * BC + wg * 32, t);
          tmem_ld_wait();
          tc_fence_before();
          // tiles left of the diagonal and inside the sequence need no mask (uniform over the warpgroup)
          const bool need_mask = (c0 + 31 > r0) || (c0 + 32 > S);
          if (need_mask) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int key = c0 + i;
              if (!(key <= row_idx && key < S)) t[i] = 0xff800000u;  // -inf
            }
          }
          float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // four independent chains
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
#pragma unroll
            for (int j = 0; j < 4; ++j) m4[j] = fmaxf(m4[j], __uint_as_float(t[i + j]));
          }
          m_loc = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
        }
        float* mx_it = mx + (it & 1) * 2 * BR;
        mx_it[wg * BR + r] = m_loc;
        named_sync_softmax();
        const float m_other = mx_it[(1 - wg) * BR + r];
        if (!step_ok) { ok = false; continue; }
        const float m_new = fmaxf(m_run, fmaxf(m_loc, m_other));
        const float alpha = exp2f((m_run - m_new) * sl2);  // first tile: m_run = -inf -> 0
        const float shift = m_new * sl2;
        float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float pi = exp2f(fmaf(__uint_as_float(t[i + j]), sl2, -shift));  // exp2(-inf) = 0 for masked entries
            l4[j] += pi;
            t[i + j] = __float_as_uint(pi);  // probabilities replace the scores in place
          }
        }
        const float l_add = (l4[0] + l4[1]) + (l4[2] + l4[3]);
        // the product of two steps ago finished long ago; its completion also frees this step's P tile
        if (it > 1 && !fold_pv(it - 2, a2)) { ok = false; continue; }
        {
          float (&pr)[32] = *reinterpret_cast<float (*)[32]>(&t[0]);
          write_e_chunk<32>((it & 1) ? e2 : e1, r, wg * 32, pr, DT);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(e_full);
        l_run = l_run * alpha + l_add;
        m_run = m_new;
        a2 = a1;
        a1 = alpha;
      }
      if (ok && n_iter > 1) ok = fold_pv(n_iter - 2, a2);
      if (ok && n_iter > 0) ok = fold_pv(n_iter - 1, a1);
      // the two partial row sums meet (both were kept relative to the same running maximum)
      float* ls = vec + 4 * BR;
      ls[wg * BR + r] = l_run;
      named_sync_softmax();
      l_run += ls[(1 - wg) * BR + r];
    }
    int stage = 0;
    for (int it = 0; it < n_iter && MODE != kFwd; ++it) {  // runs to the end even after an abandoned wait: see named_sync below
      const int c0 = (c_begin + it) * BC;  // first streamed index (key for dq, query for dkv)
      if (MODE == kDkv) {
        // stage the streamed queries' lse / dsum in shared memory (values past S are neutral)
        float* vl = vec + stage * 2 * BC;
        if (wg == 0 && r < BC) {
          const int qi = c0 + r;
          vl[r] = qi < S ? args.lse[bh * S + qi] * LOG2E : 0.f;
          vl[BC + r] = qi < S ? args.dsum[bh * S + qi] : 0.f;
        }
        named_sync_softmax();
      }
      if (!ok) { if (++stage == C::STAGES) stage = 0; continue; }
      if (!mbar_wait(t_full, it & 1, abort_flag, args.status, kKernelAttnFwd + MODE, 300)) { ok = false; if (++stage == C::STAGES) stage = 0; continue; }
      tc_fence_after();
      if (it > 0) {
        if (!mbar_wait(e_empty, (it - 1) & 1, abort_flag, args.status, kKernelAttnFwd + MODE, 310)) { ok = false; if (++stage == C::STAGES) stage = 0; continue; }
      }
      {
        const float* vl = vec + stage * 2 * BC;
        const int cw = wg * 32;  // this warpgroup's 32 columns of the step
        // only tiles that straddle the diagonal or the end of the sequence need the mask (uniform)
        const bool need_mask = (MODE == kDq) ? ((c0 + cw + 31 > r0) || (c0 + cw + 32 > S)) : ((r0 + BR - 1 > c0 + cw) || (c0 + cw + 32 > S));
        auto process = [&](auto mask_tag) {
          constexpr bool MASK = decltype(mask_tag)::value;
#pragma unroll
          for (int sub = 0; sub < 32; sub += 16) {
            const int cc = cw + sub;
            uint32_t t1[16], t2[16];
            tmem_ld_32x16(lane_addr + C::COL_T1 + cc, t1);
            tmem_ld_32x16(lane_addr + C::COL_T2 + cc, t2);
            tmem_ld_wait();
            if (sub == 16) {  // this warp holds all its scores of the step: the next score products may overwrite T1 / T2
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(t_empty);
            }
            float pv[16], ds[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int ci = c0 + cc + i;
              bool keep = true;
              float lse2, dsum;
              if (MODE == kDq) {          // row = query, column = key
                if (MASK) keep = ci <= row_idx && ci < S;
                lse2 = my_lse;
                dsum = my_dsum;
              } else {                    // row = key, column = query
                if (MASK) keep = row_idx <= ci && ci < S;
                lse2 = vl[cc + i];
                dsum = vl[BC + cc + i];
              }
              const float p = keep ? exp2f(fmaf(__uint_as_float(t1[i]), sl2, -lse2)) : 0.f;
              pv[i] = p;
              ds[i] = p * (__uint_as_float(t2[i]) - dsum) * args.scale;
            }
            if (MODE == kDq) {
              write_e_chunk<16>(e1, r, cc, ds, DT);
            } else {
              write_e_chunk<16>(e1, r, cc, pv, DT);
              write_e_chunk<16>(e2, r, cc, ds, DT);
            }
          }
        };
        if (need_mask) process(std::true_type{}); else process(std::false_type{});
        fence_proxy_async_smem();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(e_full);
      }
      if (++stage == C::STAGES) stage = 0;
    }

    // ---- final output (tcgen05.ld below is warp-wide: make the verdict warp-uniform first)
    ok = __all_sync(0xffffffffu, ok);
    if (ok && MODE != kFwd && n_iter > 0) ok = mbar_wait(acc_full, 0, abort_flag, args.status, kKernelAttnFwd + MODE, 330);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    const long long out_off = static_cast<long long>(b) * args.o_sb + static_cast<long long>(row_idx) * args.o_ss +
                              static_cast<long long>(h) * args.o_sh + col_half;
    if (MODE == kFwd) {
      if (ok && n_iter > 0 && row_idx < S) {
        const float inv = 1.f / l_run;
#pragma unroll
        for (int i = 0; i < HD; ++i) o_acc[i] *= inv;
        store_row<HD>(args.out0, out_off, o_acc, DT);
        if (wg == 0) args.lse[bh * S + row_idx] = m_run * args.scale + logf(l_run);
      }
    } else {
      // all 32 lanes of a warp take part in tcgen05.ld; rows past S are read but not stored.
      // Each warpgroup stores its half of the head dimension of every output.
#pragma unroll
      for (int which = 0; which < (MODE == kDkv ? 2 : 1); ++which) {
        float v[HD];
        if (ok && n_iter > 0) {
#pragma unroll
          for (int cc = 0; cc < HD; cc += 16) {
            uint32_t t[16];
            tmem_ld_32x16(lane_addr + (which == 0 ? C::COL_ACC1 : C::COL_ACC2) + col_half + cc, t);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) v[cc + i] = __uint_as_float(t[i]);
          }
        } else {
#pragma unroll
          for (int i = 0; i < HD; ++i) v[i] = 0.f;
        }
        if (ok && row_idx < S) store_row<HD>(which == 0 ? args.out0 : args.out1, out_off, v, DT);
      }
    }
    tc_fence_before();
  }

  __syncwarp();
  if (*abort_flag != 0u) __nanosleep(200000);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// dsum[b, h, s] = sum_d dO[b, s, h, d] * O[b, s, h, d]
template <typename T>
__global__ void dsum_kernel(const T* __restrict__ dout, const T* __restrict__ out, float* __restrict__ dsum,
                            int B, int S, int H, int DH) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;  // over B*S*H
  const long long total = static_cast<long long>(B) * S * H;
  if (idx >= total) return;
  const int hh = static_cast<int>(idx % H);
  const long long bs = idx / H;
  const int s = static_cast<int>(bs % S);
  const int bb = static_cast<int>(bs / S);
  const T* a = dout + idx * DH;
  const T* c = out + idx * DH;
  float acc = 0.f;
  for (int d = 0; d < DH; d += 8) {
    uint4 qa = *reinterpret_cast<const uint4*>(a + d), qc = *reinterpret_cast<const uint4*>(c + d);
    const T* ea = reinterpret_cast<const T*>(&qa);
    const T* ec = reinterpret_cast<const T*>(&qc);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc += static_cast<float>(ea[i]) * static_cast<float>(ec[i]);
  }
  dsum[(static_cast<long long>(bb) * H + hh) * S + s] = acc;
}

CUtensorMap map_bshd(const at::Tensor& t, int box_rows) {
  // dims innermost-first: (Dh, H, S, B)
  const uint64_t dims[4] = {static_cast<uint64_t>(t.size(3)), static_cast<uint64_t>(t.size(2)), static_cast<uint64_t>(t.size(1)),
                            static_cast<uint64_t>(t.size(0))};
  const uint64_t strides[3] = {static_cast<uint64_t>(t.stride(2)) * 2, static_cast<uint64_t>(t.stride(1)) * 2,
                               static_cast<uint64_t>(t.stride(0)) * 2};
  const uint32_t box[4] = {static_cast<uint32_t>(t.size(3)), 1, static_cast<uint32_t>(box_rows), 1};
  return make_tma_desc4(t.data_ptr(), dims, strides, box, t.size(3) == 32 ? 64 : 128);
}

void check_bshd(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.dim() == 4 && t.stride(3) == 1, name, " must be [B, S, H, Dh] with a contiguous head dim");
  TORCH_CHECK(t.scalar_type() == at::kBFloat16 || t.scalar_type() == at::kHalf, name, " must be bf16 or fp16");
  TORCH_CHECK(t.size(3) == 32 || t.size(3) == 64, "head dim must be 32 or 64");
  TORCH_CHECK(t.stride(2) % 8 == 0 && t.stride(1) % 8 == 0 && t.stride(0) % 8 == 0 && reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0,
              name, ": strides / base must be 16-byte aligned");
}

template <int DH, int MODE>
void launch(const CUtensorMap& m0, const CUtensorMap& m1, const CUtensorMap& m2, const CUtensorMap& m3, const Args& a, cudaStream_t stream) {
  using C = Cfg<DH, MODE>;
  static bool configured = false;
  if (!configured) {
    NT_CUDA_CHECK(cudaFuncSetAttribute(causal_attn_kernel<DH, MODE, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::TOTAL));
    NT_CUDA_CHECK(cudaFuncSetAttribute(causal_attn_kernel<DH, MODE, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::TOTAL));
    configured = true;
  }
  dim3 grid((a.S + BR - 1) / BR, a.H, a.B);
  if (a.dtype == 1) causal_attn_kernel<DH, MODE, 1><<<grid, THREADS, C::TOTAL, stream>>>(m0, m1, m2, m3, a);
  else causal_attn_kernel<DH, MODE, 0><<<grid, THREADS, C::TOTAL, stream>>>(m0, m1, m2, m3, a);
  NT_KERNEL_CHECK_AS(MODE == kFwd ? "causal_attn_kernel<fwd>" : (MODE == kDq ? "causal_attn_kernel<dq>" : "causal_attn_kernel<dkv>"));
}

}  // namespace attn

// q, k, v: [B, S, H, Dh] -> (out [B, S, H, Dh], lse [B, H, S] fp32)
std::vector<at::Tensor> flash_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, double scale) {
  using namespace attn;
  check_bshd(q, "q"); check_bshd(k, "k"); check_bshd(v, "v");
  TORCH_CHECK(q.sizes() == k.sizes() && q.sizes() == v.sizes() && q.scalar_type() == k.scalar_type() && q.scalar_type() == v.scalar_type(), "q, k, v must match");
  c10::cuda::CUDAGuard guard(q.device());
  const int B = q.size(0), S = q.size(1), H = q.size(2), DH = q.size(3);
  auto out = at::empty({B, S, H, DH}, q.options());
  auto lse = at::empty({B, H, S}, q.options().dtype(at::kFloat));
  if (q.numel() == 0) return {out, lse};
  Args a{};
  a.B = B; a.H = H; a.S = S; a.scale = static_cast<float>(scale);
  a.dtype = q.scalar_type() == at::kBFloat16 ? 1 : 0;
  a.out0 = out.data_ptr(); a.o_sb = out.stride(0); a.o_ss = out.stride(1); a.o_sh = out.stride(2);
  a.lse = lse.data_ptr<float>();
  a.status = device_status_word();
  const CUtensorMap mq = map_bshd(q, BR), mk = map_bshd(k, 64), mv = map_bshd(v, 64);
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  if (DH == 32) launch<32, kFwd>(mq, mq, mk, mv, a, stream); else launch<64, kFwd>(mq, mq, mk, mv, a, stream);
  return {out, lse};
}

// -> (dq, dk, dv), each [B, S, H, Dh]
// `grads`: empty, or three preallocated [B, S, H, Dh] views with identical strides (e.g. the
// thirds of one fused dQKV buffer) that receive dq, dk, dv.
std::vector<at::Tensor> flash_bwd(const at::Tensor& dout, const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                  const at::Tensor& out, const at::Tensor& lse, double scale, const std::vector<at::Tensor>& grads) {
  using namespace attn;
  check_bshd(q, "q"); check_bshd(k, "k"); check_bshd(v, "v"); check_bshd(dout, "dout"); check_bshd(out, "out");
  TORCH_CHECK(dout.is_contiguous() && out.is_contiguous(), "dout and out must be contiguous");
  c10::cuda::CUDAGuard guard(q.device());
  const int B = q.size(0), S = q.size(1), H = q.size(2), DH = q.size(3);
  at::Tensor dq, dk, dv;
  if (grads.size() == 3) {
    dq = grads[0]; dk = grads[1]; dv = grads[2];
    for (const auto& g : grads)
      TORCH_CHECK(g.sizes() == q.sizes() && g.strides() == dq.strides() && g.stride(3) == 1 && g.scalar_type() == q.scalar_type() &&
                      g.stride(2) % 8 == 0 && g.stride(1) % 8 == 0 && reinterpret_cast<uintptr_t>(g.data_ptr()) % 16 == 0,
                  "flash_bwd: gradient outputs must be same-strided, 16-byte aligned [B, S, H, Dh] views");
  } else {
    TORCH_CHECK(grads.empty(), "flash_bwd: pass zero or three gradient outputs");
    dq = at::empty({B, S, H, DH}, q.options());
    dk = at::empty({B, S, H, DH}, q.options());
    dv = at::empty({B, S, H, DH}, q.options());
  }
  if (q.numel() == 0) return {dq, dk, dv};
  auto dsum = at::empty({B, H, S}, lse.options());
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  const long long rows = static_cast<long long>(B) * S * H;
  if (q.scalar_type() == at::kBFloat16)
    dsum_kernel<__nv_bfloat16><<<static_cast<unsigned>((rows + 255) / 256), 256, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(dout.data_ptr()), reinterpret_cast<const __nv_bfloat16*>(out.data_ptr()), dsum.data_ptr<float>(), B, S, H, DH);
  else
    dsum_kernel<__half><<<static_cast<unsigned>((rows + 255) / 256), 256, 0, stream>>>(
        reinterpret_cast<const __half*>(dout.data_ptr()), reinterpret_cast<const __half*>(out.data_ptr()), dsum.data_ptr<float>(), B, S, H, DH);
  NT_KERNEL_CHECK();
  Args a{};
  a.B = B; a.H = H; a.S = S; a.scale = static_cast<float>(scale);
  a.dtype = q.scalar_type() == at::kBFloat16 ? 1 : 0;
  a.o_sb = dq.stride(0); a.o_ss = dq.stride(1); a.o_sh = dq.stride(2);
  a.lse = const_cast<float*>(lse.data_ptr<float>());
  a.dsum = dsum.data_ptr<float>();
  a.status = device_status_word();
  // dQ pass: resident (Q, dO), streamed (K, V)
  {
    Args d = a;
    d.out0 = dq.data_ptr();
    const CUtensorMap r0 = map_bshd(q, BR), r1 = map_bshd(dout, BR), c0 = map_bshd(k, 64), c1 = map_bshd(v, 64);
    if (DH == 32) launch<32, kDq>(r0, r1, c0, c1, d, stream); else launch<64, kDq>(r0, r1, c0, c1, d, stream);
  }
  // dK/dV pass: resident (K, V), streamed (Q, dO)
  {
    Args d = a;
    d.out0 = dv.data_ptr();
    d.out1 = dk.data_ptr();
    const CUtensorMap r0 = map_bshd(k, BR), r1 = map_bshd(v, BR), c0 = map_bshd(q, 64), c1 = map_bshd(dout, 64);
    if (DH == 32) launch<32, kDkv>(r0, r1, c0, c1, d, stream); else launch<64, kDkv>(r0, r1, c0, c1, d, stream);
  }
  return {dq, dk, dv};
}

}  // namespace nt
