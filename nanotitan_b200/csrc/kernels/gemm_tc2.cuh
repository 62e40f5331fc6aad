// CTA-pair variant of the tcgen05 GEMM: two CTAs of a cluster compute one 256 x 256 tile with
// `tcgen05.mma.cta_group::2`.  Each CTA loads its own 128 rows of A and its own 128 columns of B
// (so a byte of B crosses L2 -> shared memory once per pair instead of once per CTA, and a stage is
// 32 KB instead of 48 KB: six stages in flight instead of four), the leader CTA issues the MMAs for
// both, and each CTA drains its own 128 TMEM lanes.  Cross-CTA signalling: the peer's TMA loads
// count their bytes on the leader's "full" barrier, `tcgen05.commit` fans its arrival out to both
// CTAs' "empty" / "accumulator ready" barriers, and the peer's epilogue warps arrive on the
// leader's "accumulator free" barrier through its cluster address.  No TMA load uses multicast.
//
// Covers the dense and grouped-M problem shapes with all epilogues of gemm_tc.cuh; the ragged
// reductions (grouped-K, which must patch operand tiles in shared memory) stay on the one-CTA kernel.
#pragma once
#include "gemm_tc.cuh"

namespace nt {
namespace gemm {

constexpr int PAIR_BM = 256;   // rows per pair tile
constexpr int PAIR_BN = 256;   // accumulator columns per tile
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_B_BYTES = (PAIR_BN / 2) * BK * 2;  // this CTA's half of B per stage
constexpr int PAIR_STAGE_BYTES = A_STAGE_BYTES + PAIR_B_BYTES;
constexpr int PAIR_SMEM = PAIR_STAGES * PAIR_STAGE_BYTES + STAGING_BYTES + (2 * PAIR_STAGES + 4) * 8 + 16 + (MAX_GROUPS + 1) * 4 + 1024;

template <int EPI>
__device__ __forceinline__ int pair_total_tiles(const Args& a, const int* tile_start) {
  const int n_tiles = ceil_div(a.N, tile_n<PAIR_BN, EPI>());
  if (a.mode == kDense) return ceil_div(a.M, PAIR_BM) * n_tiles;
  return tile_start[a.G] * n_tiles;
}

// Tile of the *pair*; a CTA's own rows start at m0 + 128 * rank.
template <int EPI>
__device__ __forceinline__ Tile pair_get_tile(const Args& a, const int* tile_start, int t, int rank) {
  Tile ti;
  const int tn = tile_n<PAIR_BN, EPI>();
  const int n_tiles = ceil_div(a.N, tn);
  const int nt = t % n_tiles, mt = t / n_tiles;
  ti.n0 = nt * tn;
  ti.split = 0; ti.k_row0 = 0; ti.k_rows = 0;
  ti.k_chunks = ceil_div(a.K, BK);
  int seg_end;
  if (a.mode == kDense) {
    ti.g = 0;
    ti.m0 = mt * PAIR_BM + rank * BM;
    seg_end = a.M;
  } else {
    int g = 0;
    while (g + 1 < a.G && tile_start[g + 1] <= mt) ++g;
    ti.g = g;
    ti.m0 = a.offsets[g] + (mt - tile_start[g]) * PAIR_BM + rank * BM;
    seg_end = a.offsets[g + 1];
  }
  ti.rows_valid = max(0, min(BM, seg_end - ti.m0));
  return ti;
}

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB0,
                    const __grid_constant__ CUtensorMap tmB1, const __grid_constant__ CUtensorMap tmB2,
                    const __grid_constant__ CUtensorMap tmC0, const __grid_constant__ CUtensorMap tmC1,
                    const __grid_constant__ CUtensorMap tmC2, const Args args) {
  using namespace sm100;
  constexpr int BN = PAIR_BN;
  constexpr int STAGES = PAIR_STAGES;
  constexpr uint32_t TMEM_COLS = 512;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + STAGES * PAIR_STAGE_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(staging + STAGING_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  int* tile_start = reinterpret_cast<int*>(tmem_slot + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = static_cast<int>(cluster_ctarank());
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&tmem_full[i], 1); mbar_init(&tmem_empty[i], 2 * EPI_WARPS); }  // both CTAs' epilogue warps
    *abort_flag = 0u;
    fence_barrier_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB0);
    if (args.b_split != kBNone) prefetch_tmap(&tmB1);
    tile_start[0] = 0;
    if (args.mode == kGroupedM) {
      int acc = 0;
      for (int g = 0; g < args.G; ++g) {
        acc += ceil_div(args.offsets[g + 1] - args.offsets[g], PAIR_BM);
        tile_start[g + 1] = acc;
      }
    }
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anything signals across the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const bool dead = args.status != nullptr && *reinterpret_cast<volatile uint32_t*>(&args.status->code) != 0u;
  const int n_total = dead ? 0 : pair_total_tiles<EPI>(args, tile_start);
  const int pair_id = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const uint32_t idesc = umma_idesc(args.dtype, PAIR_BM, BN, args.a_mn, args.b_mn);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = pair_id; t < n_total && ok; t += n_pairs) {
        const Tile ti = pair_get_tile<EPI>(args, tile_start, t, rank);
        for (int kc = 0; kc < ti.k_chunks; ++kc) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, args.status, kKernelGemm, 100 + stage)) { ok = false; break; }
          uint8_t* sA = smem + stage * PAIR_STAGE_BYTES;
          uint8_t* sB = sA + A_STAGE_BYTES;
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * PAIR_STAGE_BYTES);  // both CTAs' bytes land on the leader's barrier
          const uint32_t bar = smem_u32(&full_bar[stage]) & 0xFEFFFFFFu;        // the leader's copy of this barrier
          const int kk = kc * BK;
          if (!args.a_mn) {
            tma_load_2d_pair(sA, &tmA, bar, kk, ti.m0);
          } else {
            tma_load_2d_pair(sA, &tmA, bar, ti.m0, kk);
            tma_load_2d_pair(sA + 8192, &tmA, bar, ti.m0 + 64, kk);
          }
          const int gb = (args.mode == kGroupedM) ? ti.g : 0;
          const CUtensorMap* mp = &tmB0;
          int nb = ti.n0 + rank * (BN / 2), kcoord = kk;
          if (args.b_split == kBDual) {           // this CTA's half: gate (rank 0) or value (rank 1)
            mp = rank == 0 ? &tmB0 : &tmB1;
            nb = ti.n0;
          } else if (args.b_split == kBSplitN) {
            const int src = ti.n0 / args.b_split_size;
            mp = src == 0 ? &tmB0 : (src == 1 ? &tmB1 : &tmB2);
            nb -= src * args.b_split_size;
          } else if (args.b_split == kBSplitK) {
            const int src = kk / args.b_split_size;
            mp = src == 0 ? &tmB0 : (src == 1 ? &tmB1 : &tmB2);
            kcoord = kk - src * args.b_split_size;
          }
          if (!args.b_mn) {
            tma_load_3d_pair(sB, mp, bar, kcoord, nb, gb);
          } else {
            tma_load_3d_pair(sB, mp, bar, nb, kcoord, gb);
            tma_load_3d_pair(sB + 8192, mp, bar, nb + 64, kcoord, gb);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (leader) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int t = pair_id; t < n_total && ok; t += n_pairs) {
        const Tile ti = pair_get_tile<EPI>(args, tile_start, t, rank);
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1u, abort_flag, args.status, kKernelGemm, 200 + acc)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kc = 0; kc < ti.k_chunks; ++kc) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, args.status, kKernelGemm, 300 + stage)) { ok = false; break; }
          tc_fence_after();
          if (lane == 0) {
            const uint32_t a_addr = smem_u32(smem + stage * PAIR_STAGE_BYTES), b_addr = a_addr + A_STAGE_BYTES;
#pragma unroll
            for (int ks = 0; ks < BK / 16; ++ks) {
              const uint64_t da = args.a_mn ? smem_desc_sw128(a_addr + ks * 2048, 8192, 1024) : smem_desc_sw128(a_addr + ks * 32, 16, 1024);
              const uint64_t db = args.b_mn ? smem_desc_sw128(b_addr + ks * 2048, 8192, 1024) : smem_desc_sw128(b_addr + ks * 32, 16, 1024);
              umma_f16_pair(d_tmem, da, db, idesc, (kc | ks) != 0 ? 1u : 0u);
            }
            umma_commit_pair(&empty_bar[stage], 3);
            if (kc == ti.k_chunks - 1) umma_commit_pair(&tmem_full[acc], 3);
          }
          __syncwarp();
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9 of both CTAs)
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    constexpr int SPAN = (EPI == kEpiSwigluFwd ? BN / 2 : BN) / 2;
    const int c_lo = half * SPAN, c_hi = c_lo + SPAN;
    const int row_in_tile = quarter * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    Stager st;
    st.slots = staging + (warp - 2) * STAGING_WARP_BYTES;
    st.map0 = &tmC0; st.map1 = &tmC1; st.map2 = &tmC2;
    st.next = 0;
    st.lane = lane;
    for (int t = pair_id; t < n_total && ok; t += n_pairs) {
      const Tile ti = pair_get_tile<EPI>(args, tile_start, t, rank);
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag, args.status, kKernelGemm, 400 + acc)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + static_cast<uint32_t>(acc * BN) + (static_cast<uint32_t>(quarter * 32) << 16);
      const bool row_ok = row_in_tile < ti.rows_valid;
      const long long row = static_cast<long long>(ti.m0) + row_in_tile;
      const int warp_rows = max(0, min(32, ti.rows_valid - quarter * 32));
      st.on = args.c_tma != 0 && warp_rows > 0 && (args.mode == kDense || warp_rows == 32);
      st.row0 = ti.m0 + quarter * 32;
      epilogue_rows<BN, EPI>(args, ti, t_addr, row_ok, true, row, c_lo, c_hi, st);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(map_to_cta(smem_u32(&tmem_empty[acc]), 0));  // the leader's barrier
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (lane == 0) tma_store_wait_read<0>();
  }

  // ---------------------------------------------------------------------- teardown
  __syncwarp();
  if (*abort_flag != 0u) __nanosleep(200000);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the leader's MMAs read the peer's shared memory: nobody leaves early
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

}  // namespace gemm
}  // namespace nt
