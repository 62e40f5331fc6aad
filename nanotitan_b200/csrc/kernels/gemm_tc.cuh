// Persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   C[128 x BN tile] = A[128 x K] * B[BN x K]^T, bf16/fp16 operands, fp32 accumulation in TMEM.
//
// One CTA per SM walks a list of output tiles.  Warp 0 feeds a ring of shared-memory stages
// with TMA (128-byte swizzle, no multicast); warp 1 issues `tcgen05.mma` (one elected lane)
// into one of two TMEM accumulators and signals stage release / accumulator-ready through
// `tcgen05.commit`; warps 2-9 drain the other accumulator with `tcgen05.ld`, apply the
// epilogue and store (through shared memory and TMA), so the epilogue of tile i overlaps the
// MMAs of tile i+1.
//
// Either operand may be K-major (reduction dim contiguous) or MN-major; B may come from up to
// three tensors (split along N, along K, or as two half-tiles for SwiGLU), C may be split along
// N over up to three tensors.  Three problem shapes share the kernel:
//   dense      one problem;
//   grouped-M  rows of A/C are segmented by `offsets`, segment g multiplies B[g] (expert
//              forward and dgrad; tiles never mix experts, partial tiles are row-masked);
//   grouped-K  the reduction dim is segmented, segment g produces C[g] (expert wgrad; the
//              ragged last chunk of a segment is zeroed in shared memory before the MMA).
// Every mbarrier wait is bounded; a wait that runs out raises the CTA's abort flag, records a
// status word and lets the kernel run to its end, where TMEM is released.
#pragma once
#include "sm100.cuh"

namespace nt {
namespace gemm {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int MAX_GROUPS = 256;
constexpr int EPI_WARPS = 8;                      // two per scheduler: one warp's dependent chains hide behind the other's
constexpr int NUM_THREADS = 64 + 32 * EPI_WARPS;  // TMA warp, MMA warp, epilogue warps
constexpr int STAGING_SLOT_BYTES = 32 * 64;               // 32 rows x 32 16-bit columns
constexpr int STAGING_WARP_BYTES = 2 * STAGING_SLOT_BYTES;  // per epilogue warp
constexpr int STAGING_BYTES = EPI_WARPS * STAGING_WARP_BYTES;

enum Mode : int { kDense = 0, kGroupedM = 1, kGroupedK = 2 };
enum BSplit : int { kBNone = 0, kBSplitN = 1, kBSplitK = 2, kBDual = 3 };
enum Epilogue : int { kEpiStore = 0, kEpiSwigluFwd = 1, kEpiSwigluBwd = 2 };

struct Args {
  int M, N, K;  // dense: the problem.  grouped-M: M = total rows.  grouped-K: M, N of every C[g]
  int mode, G;
  const int* offsets;  // [G+1] row offsets (grouped modes)
  int a_mn, b_mn;      // 1 = MN-major operand
  int dtype;           // 0 = fp16, 1 = bf16
  int b_split, b_split_size;
  int c_split_size;  // 0 = single destination, else columns per destination
  void* C[3];
  long long ldc, c_group_stride;  // elements
  int out_f32, accumulate;
  const void* R;  // kEpiStore: residual added to the tile (operand dtype) or null.  kEpiSwigluBwd: GV
  long long ldr;
  void* C2;  // kEpiSwigluFwd: H output
  long long ldc2;
  // grouped-K only: every segment's reduction is cut into `k_splits` parts whose fp32 partial
  // tiles go to `ws` ([k_splits][G][M][N]); a second kernel folds them in a fixed order.
  int k_splits;
  float* ws;
  int c_tma;  // 1: the C tensor maps are valid and full 32-row groups may use staged TMA stores
  StatusWord* status;
};

struct Tile {
  int split;       // grouped-K: which part of the segment's reduction
  int g;           // group
  int m0;          // first row of the tile: A/C row (dense, grouped-M) or C[g] row (grouped-K)
  int rows_valid;  // rows of the tile that exist
  int n0;          // first output column
  int k_chunks;    // BK-sized steps of the reduction
  int k_row0;      // grouped-K: first row of the segment in A/B
  int k_rows;      // grouped-K: rows in the segment
};

template <int BN>
struct Smem {
  static constexpr int B_STAGE_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
  static constexpr int BAR_BYTES = (2 * STAGES + 4) * 8;
  static constexpr int EXTRA_BYTES = 16 + (MAX_GROUPS + 1) * 4;
  static constexpr int TOTAL = TILE_BYTES + STAGING_BYTES + BAR_BYTES + EXTRA_BYTES + 1024;  // + alignment slack
};

__device__ __forceinline__ int ceil_div(int a, int b) { return (a + b - 1) / b; }

// n-extent covered by one tile in output columns (SwiGLU-forward tiles hold gate|val halves).
template <int BN, int EPI>
__device__ __forceinline__ constexpr int tile_n() {
  return EPI == kEpiSwigluFwd ? BN / 2 : BN;
}

template <int BN, int EPI>
__device__ __forceinline__ int total_tiles(const Args& a, const int* tile_start) {
  const int n_tiles = ceil_div(a.N, tile_n<BN, EPI>());
  if (a.mode == kDense) return ceil_div(a.M, BM) * n_tiles;
  if (a.mode == kGroupedM) return tile_start[a.G] * n_tiles;
  return a.k_splits * a.G * ceil_div(a.M, BM) * n_tiles;
}

template <int BN, int EPI>
__device__ __forceinline__ Tile get_tile(const Args& a, const int* tile_start, int t) {
  Tile ti;
  const int tn = tile_n<BN, EPI>();
  const int n_tiles = ceil_div(a.N, tn);
  const int nt = t % n_tiles;
  const int mt = t / n_tiles;
  ti.n0 = nt * tn;
  ti.k_row0 = 0;
  ti.k_rows = 0;
  ti.split = 0;
  if (a.mode == kDense) {
    ti.g = 0;
    ti.m0 = mt * BM;
    ti.rows_valid = min(BM, a.M - ti.m0);
    ti.k_chunks = ceil_div(a.K, BK);
  } else if (a.mode == kGroupedM) {
    int g = 0;
    while (g + 1 < a.G && tile_start[g + 1] <= mt) ++g;
    const int seg0 = a.offsets[g], seg1 = a.offsets[g + 1];
    ti.g = g;
    ti.m0 = seg0 + (mt - tile_start[g]) * BM;
    ti.rows_valid = min(BM, seg1 - ti.m0);
    ti.k_chunks = ceil_div(a.K, BK);
  } else {
    const int m_tiles = ceil_div(a.M, BM);
    const int sg = mt / m_tiles;  // split-major, then group
    ti.split = sg / a.G;
    ti.g = sg - ti.split * a.G;
    ti.m0 = (mt % m_tiles) * BM;
    ti.rows_valid = min(BM, a.M - ti.m0);
    const int seg0 = a.offsets[ti.g];
    const int seg_rows = a.offsets[ti.g + 1] - seg0;
    const int chunks_total = ceil_div(seg_rows, BK);
    const int per_split = ceil_div(chunks_total, a.k_splits);
    const int chunk0 = ti.split * per_split;
    ti.k_chunks = max(0, min(per_split, chunks_total - chunk0));
    ti.k_row0 = seg0 + chunk0 * BK;
    ti.k_rows = max(0, seg_rows - chunk0 * BK);  // rows from this part's start to the segment's end
  }
  return ti;
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }

__device__ __forceinline__ uint32_t pack2(float lo, float hi, int dtype) {
  if (dtype == 1) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void unpack2(uint32_t w, int dtype, float& lo, float& hi) {
  if (dtype == 1) {
    float2 f = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w));
    lo = f.x; hi = f.y;
  } else {
    float2 f = __half22float2(*reinterpret_cast<__half2*>(&w));
    lo = f.x; hi = f.y;
  }
}

// Load up to 32 consecutive 16-bit elements of one row as floats (zeros past `valid`).
__device__ __forceinline__ void load_row32(const void* base, long long elem_off, int valid, int dtype, float (&out)[32]) {
  const uint16_t* p = reinterpret_cast<const uint16_t*>(base) + elem_off;
  const bool vec = valid == 32 && (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
  if (vec) {
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      uint4 q = __ldg(reinterpret_cast<const uint4*>(p) + v);
      unpack2(q.x, dtype, out[v * 8 + 0], out[v * 8 + 1]);
      unpack2(q.y, dtype, out[v * 8 + 2], out[v * 8 + 3]);
      unpack2(q.z, dtype, out[v * 8 + 4], out[v * 8 + 5]);
      unpack2(q.w, dtype, out[v * 8 + 6], out[v * 8 + 7]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      float f = 0.f;
      if (i < valid) {
        uint16_t raw = p[i];
        f = dtype == 1 ? __bfloat162float(*reinterpret_cast<__nv_bfloat16*>(&raw))
                       : __half2float(*reinterpret_cast<__half*>(&raw));
      }
      out[i] = f;
    }
  }
}

// Store up to 32 consecutive values of one row as 16-bit (dtype) or fp32 elements.
__device__ __forceinline__ void store_row32(void* base, long long elem_off, int valid, int dtype, bool f32, const float (&v)[32]) {
  if (valid <= 0) return;
  if (f32) {
    float* p = reinterpret_cast<float*>(base) + elem_off;
    if (valid == 32 && (reinterpret_cast<uintptr_t>(p) & 15u) == 0) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        reinterpret_cast<float4*>(p)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i < valid) p[i] = v[i];
    }
    return;
  }
  uint16_t* p = reinterpret_cast<uint16_t*>(base) + elem_off;
  if (valid == 32 && (reinterpret_cast<uintptr_t>(p) & 15u) == 0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 q;
      q.x = pack2(v[8 * i + 0], v[8 * i + 1], dtype);
      q.y = pack2(v[8 * i + 2], v[8 * i + 3], dtype);
      q.z = pack2(v[8 * i + 4], v[8 * i + 5], dtype);
      q.w = pack2(v[8 * i + 6], v[8 * i + 7], dtype);
      reinterpret_cast<uint4*>(p)[i] = q;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      if (i < valid) {
        uint32_t w = pack2(v[i], 0.f, dtype);
        p[i] = static_cast<uint16_t>(w & 0xFFFFu);
      }
    }
  }
}

// ---- staged stores -------------------------------------------------------------------------
// A thread of an epilogue warp owns one row of the accumulator, so direct stores make every warp
// store instruction touch 32 different rows (32 half-used sectors per instruction, and the LSU
// becomes the bottleneck of short-K problems).  Instead each warp owns two 2 KB slots of shared
// memory; a 32 row x 32 column chunk is written there (one conflict-free 64-byte row per lane,
// in the layout of a SWIZZLE_64B tensor map) and one lane hands it to the TMA engine, which
// writes full 64-byte row segments and clips at the tensor's edges.  A slot is rewritten only
// after the store group that last read it has finished reading.
struct Stager {
  uint8_t* slots;                          // this warp's two slots
  const CUtensorMap *map0, *map1, *map2;  // destinations (the host side says which is which per epilogue)
  int next;                                // ring position (store epilogue)
  int lane;
  int row0;                                // per tile: global row of the warp's first accumulator lane
  bool on;                                 // per tile: this warp's rows go through the slots (else direct stores)
};

// 32 floats -> 16 words of the storage dtype; the dtype test is one uniform branch per chunk.
__device__ __forceinline__ void pack32(const float (&v)[32], int dtype, uint32_t (&w)[16]) {
  if (dtype == 1) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      __nv_bfloat162 t = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&t);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      __half2 t = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&t);
    }
  }
}
// 32 stored values (four 16-byte pieces) -> floats.
__device__ __forceinline__ void unpack32(const uint4 (&q)[4], int dtype, float (&out)[32]) {
  const uint32_t* w = reinterpret_cast<const uint32_t*>(q);
  if (dtype == 1) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
      out[2 * i] = f.x; out[2 * i + 1] = f.y;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      out[2 * i] = f.x; out[2 * i + 1] = f.y;
    }
  }
}

// This lane's row (32 x 16 bit) into a slot: 16-byte piece j of row r sits at piece j ^ ((r >> 1) & 3).
__device__ __forceinline__ void stage_row(uint8_t* slot, int lane, const uint32_t (&w)[16]) {
  const uint32_t base = sm100::smem_u32(slot) + static_cast<uint32_t>(lane) * 64u;
  const uint32_t sw = (static_cast<uint32_t>(lane) >> 1) & 3u;
#pragma unroll
  for (uint32_t j = 0; j < 4; ++j) sm100::st_shared_v4(base + ((j ^ sw) << 4), w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
}

// Before a slot is rewritten: at most PENDING earlier store groups of this warp may still be reading.
template <int PENDING>
__device__ __forceinline__ void stager_acquire(const Stager& st) {
  if (st.lane == 0) sm100::tma_store_wait_read<PENDING>();
  __syncwarp();
}
// After the rows are written: make them visible to the TMA engine.
__device__ __forceinline__ void stager_publish() {
  sm100::fence_proxy_async_smem();
  __syncwarp();
}

// Drains this warp's share of one accumulator tile through the epilogue EPI: its 32 TMEM lanes
// (= 32 rows) of accumulator columns [c_lo, c_hi) (multiples of 32; for the SwiGLU forward the
// range counts output columns, each of which has a gate and a value accumulator column).
// `t_addr`: TMEM address of the tile's first column in this warp's lanes; `row`: global row of
// this thread; `row_ok`: the row exists; `have_acc`: the tile had at least one reduction step.
template <int BN, int EPI>
__device__ __forceinline__ void epilogue_rows(const Args& args, const Tile& ti, uint32_t t_addr, bool row_ok, bool have_acc, long long row,
                                              int c_lo, int c_hi, Stager& st) {
  using namespace sm100;
  if constexpr (EPI == kEpiStore) {
    const long long grp_off = (args.mode == kGroupedK) ? static_cast<long long>(ti.g) * args.c_group_stride : 0;
    const bool partial = args.mode == kGroupedK && args.k_splits > 1;
    float* ws_tile = partial ? args.ws + (static_cast<long long>(ti.split) * args.G + ti.g) * args.M * args.N : nullptr;
    // Residual rows are requested one chunk ahead so their latency hides behind the previous chunk.
    const uint16_t* r_row = reinterpret_cast<const uint16_t*>(args.R) + row * args.ldr;
    const bool fast_r = args.R != nullptr && row_ok && (reinterpret_cast<uintptr_t>(r_row) & 15u) == 0;
    uint4 rq[4];
    auto fetch_r = [&](int col) {
      if (fast_r && col + 32 <= args.N && col < ti.n0 + c_hi) {
#pragma unroll
        for (int q = 0; q < 4; ++q) rq[q] = __ldg(reinterpret_cast<const uint4*>(r_row + col) + q);
      }
    };
    fetch_r(ti.n0 + c_lo);
    // One 32-column chunk: epilogue math on the raw accumulator words, then the store.
    auto process = [&](int c0, uint32_t (&r)[32]) {
      const int col = ti.n0 + c0;
      if (!have_acc) {  // uniform; only the ragged reductions have empty tiles
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = 0u;
      }
      float v[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
      const int valid = min(32, args.N - col);
      if (row_ok && partial) {
        store_row32(ws_tile, row * args.N + col, valid, args.dtype, true, v);
        return;
      }
      if (args.R != nullptr) {
        if (fast_r && valid == 32) {
          float rr[32];
          unpack32(rq, args.dtype, rr);
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] += rr[i];
        } else if (row_ok) {
          float rr[32];
          load_row32(args.R, row * args.ldr + col, valid, args.dtype, rr);
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] += rr[i];
        }
        fetch_r(col + 32);  // the next chunk's residual is in flight during this chunk's stores
      }
      void* dst = args.C[0];
      int dcol = col, d = 0;
      if (args.c_split_size > 0) {
        d = col / args.c_split_size;
        dst = args.C[d];
        dcol = col - d * args.c_split_size;
      }
      const long long off = grp_off + row * args.ldc + dcol;
      if (row_ok && args.accumulate) {
        if (args.out_f32) {
          const float* p = reinterpret_cast<const float*>(dst) + off;
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (i < valid) v[i] += p[i];
        } else {
          float old[32];
          load_row32(dst, off, valid, args.dtype, old);
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] += old[i];
        }
      }
      if (st.on) {
        uint32_t w[16];
        pack32(v, args.dtype, w);
        stager_acquire<1>(st);
        uint8_t* slot = st.slots + st.next * STAGING_SLOT_BYTES;
        stage_row(slot, st.lane, w);
        stager_publish();
        if (st.lane == 0) {
          tma_store_2d(d == 0 ? st.map0 : (d == 1 ? st.map1 : st.map2), slot, dcol, st.row0);
          tma_store_commit();
        }
        st.next ^= 1;
      } else if (row_ok) {
        store_row32(dst, off, valid, args.dtype, args.out_f32 != 0, v);
      }
    };
    // Chunks that start inside the matrix; the TMEM read of chunk c+1 is in flight during chunk c.
    const int c_begin = c_lo / 32;
    const int c_end = min(c_hi / 32, (args.N - ti.n0 + 31) / 32);
    uint32_t ra[32], rb[32];
    if (have_acc && c_begin < c_end) tmem_ld_32x32(t_addr + c_begin * 32, ra);
#pragma unroll 1
    for (int c = c_begin; c < c_end; c += 2) {
      if (have_acc) {
        tmem_ld_wait_on(ra);
        if (c + 1 < c_end) tmem_ld_32x32(t_addr + (c + 1) * 32, rb);
      }
      process(c * 32, ra);
      if (c + 1 < c_end) {
        if (have_acc) {
          tmem_ld_wait_on(rb);
          if (c + 2 < c_end) tmem_ld_32x32(t_addr + (c + 2) * 32, ra);
        }
        process((c + 1) * 32, rb);
      }
    }
  } else if constexpr (EPI == kEpiSwigluFwd) {
    // accumulator columns [0, BN/2) = gate, [BN/2, BN) = value, for output columns n0 .. n0+BN/2
#pragma unroll 1
    for (int c0 = c_lo; c0 < c_hi; c0 += 32) {
      const int col = ti.n0 + c0;
      if (col >= args.N) break;
      uint32_t rg[32], rv[32];
      tmem_ld_32x32(t_addr + c0, rg);
      tmem_ld_32x32(t_addr + BN / 2 + c0, rv);
      tmem_ld_wait();
      if (!st.on && !row_ok) continue;
      const int valid = min(32, args.N - col);
      float g[32], u[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        g[i] = __uint_as_float(rg[i]);
        u[i] = __uint_as_float(rv[i]);
      }
      if (st.on) {
        // gate and value chunks fill the two slots and leave; h is computed while the TMA engine
        // reads them and then reuses the first slot
        uint32_t w[16];
        stager_acquire<0>(st);
        pack32(g, args.dtype, w);
        stage_row(st.slots, st.lane, w);
        pack32(u, args.dtype, w);
        stage_row(st.slots + STAGING_SLOT_BYTES, st.lane, w);
        stager_publish();
        if (st.lane == 0) {
          tma_store_2d(st.map0, st.slots, col, st.row0);
          tma_store_commit();
          tma_store_2d(st.map0, st.slots + STAGING_SLOT_BYTES, args.N + col, st.row0);
          tma_store_commit();
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) g[i] = silu_f(g[i]) * u[i];
        pack32(g, args.dtype, w);
        stager_acquire<1>(st);  // the gate store has read the first slot
        stage_row(st.slots, st.lane, w);
        stager_publish();
        if (st.lane == 0) {
          tma_store_2d(st.map1, st.slots, col, st.row0);
          tma_store_commit();
        }
      } else {
        float h[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) h[i] = silu_f(g[i]) * u[i];
        store_row32(args.C[0], row * args.ldc + col, valid, args.dtype, false, g);
        store_row32(args.C[0], row * args.ldc + args.N + col, valid, args.dtype, false, u);
        store_row32(args.C2, row * args.ldc2 + col, valid, args.dtype, false, h);
      }
    }
  } else {
    // kEpiSwigluBwd: accumulator = dH tile; R = GV [rows, 2N]; C[0] = dGV [rows, 2N].
    // The gate / value rows of chunk c+1 are requested before chunk c is processed, so their
    // memory latency overlaps the TMEM read and the math instead of stalling every chunk.
    const uint16_t* gv_row = reinterpret_cast<const uint16_t*>(args.R) + row * args.ldr;
    const bool fast = row_ok && (reinterpret_cast<uintptr_t>(gv_row) & 15u) == 0 && (args.N % 8) == 0;
    uint4 gq[4], uq[4];
    auto fetch = [&](int col) {
      if (fast && col + 32 <= args.N) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          gq[v] = __ldg(reinterpret_cast<const uint4*>(gv_row + col) + v);
          uq[v] = __ldg(reinterpret_cast<const uint4*>(gv_row + args.N + col) + v);
        }
      }
    };
    fetch(ti.n0 + c_lo);
#pragma unroll 1
    for (int c0 = c_lo; c0 < c_hi; c0 += 32) {
      const int col = ti.n0 + c0;
      if (col >= args.N) break;
      uint32_t r[32];
      tmem_ld_32x32(t_addr + c0, r);
      float g[32], u[32];
      const int valid = min(32, args.N - col);
      if (fast && valid == 32) {
        unpack32(gq, args.dtype, g);
        unpack32(uq, args.dtype, u);
      } else if (row_ok) {
        load_row32(args.R, row * args.ldr + col, valid, args.dtype, g);
        load_row32(args.R, row * args.ldr + args.N + col, valid, args.dtype, u);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) { g[i] = 0.f; u[i] = 0.f; }
      }
      if (c0 + 32 < c_hi) fetch(col + 32);  // next chunk's rows are in flight during this chunk's math
      tmem_ld_wait();
      if (!st.on && !row_ok) continue;
      float dg[32], du[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float dh = __uint_as_float(r[i]);
        const float sig = 1.f / (1.f + __expf(-g[i]));
        const float sl = g[i] * sig;
        dg[i] = dh * u[i] * (sig * (1.f + g[i] * (1.f - sig)));
        du[i] = dh * sl;
      }
      if (st.on) {
        uint32_t w[16];
        stager_acquire<0>(st);
        pack32(dg, args.dtype, w);
        stage_row(st.slots, st.lane, w);
        pack32(du, args.dtype, w);
        stage_row(st.slots + STAGING_SLOT_BYTES, st.lane, w);
        stager_publish();
        if (st.lane == 0) {
          tma_store_2d(st.map0, st.slots, col, st.row0);
          tma_store_2d(st.map0, st.slots + STAGING_SLOT_BYTES, args.N + col, st.row0);
          tma_store_commit();
        }
      } else {
        store_row32(args.C[0], row * args.ldc + col, valid, args.dtype, false, dg);
        store_row32(args.C[0], row * args.ldc + args.N + col, valid, args.dtype, false, du);
      }
    }
  }
}

template <int BN, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB0,
               const __grid_constant__ CUtensorMap tmB1, const __grid_constant__ CUtensorMap tmB2,
               const __grid_constant__ CUtensorMap tmC0, const __grid_constant__ CUtensorMap tmC1,
               const __grid_constant__ CUtensorMap tmC2, const Args args) {
  using namespace sm100;
  using S = Smem<BN>;
  constexpr int STAGES = S::STAGES;
  constexpr uint32_t TMEM_COLS = 2 * BN;  // two accumulators; 128, 256 or 512 columns

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + S::TILE_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(staging + STAGING_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  int* tile_start = reinterpret_cast<int*>(tmem_slot + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], EPI_WARPS);
    }
    *abort_flag = 0u;
    fence_barrier_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB0);
    if (args.b_split != kBNone) prefetch_tmap(&tmB1);
    tile_start[0] = 0;
    if (args.mode == kGroupedM) {
      int acc = 0;
      for (int g = 0; g < args.G; ++g) {
        acc += ceil_div(args.offsets[g + 1] - args.offsets[g], BM);
        tile_start[g + 1] = acc;
      }
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // a failure recorded earlier (by any kernel) turns every later CTA into a no-op until the host clears it
  const bool dead = args.status != nullptr && *reinterpret_cast<volatile uint32_t*>(&args.status->code) != 0u;
  const int n_total = dead ? 0 : total_tiles<BN, EPI>(args, tile_start);
  const uint32_t idesc = umma_idesc(args.dtype, BM, BN, args.a_mn, args.b_mn);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < n_total && ok; t += gridDim.x) {
        const Tile ti = get_tile<BN, EPI>(args, tile_start, t);
        for (int kc = 0; kc < ti.k_chunks; ++kc) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, args.status, kKernelGemm, 100 + stage)) { ok = false; break; }
          uint8_t* sA = smem + stage * S::STAGE_BYTES;
          uint8_t* sB = sA + A_STAGE_BYTES;
          mbar_expect_tx(&full_bar[stage], S::STAGE_BYTES);
          const int kk = kc * BK;
          // ---- A
          if (!args.a_mn) {
            tma_load_2d(sA, &tmA, &full_bar[stage], kk, ti.m0);
          } else {
            const int krow = ti.k_row0 + kk;
            tma_load_2d(sA, &tmA, &full_bar[stage], ti.m0, krow);
            tma_load_2d(sA + 8192, &tmA, &full_bar[stage], ti.m0 + 64, krow);
          }
          // ---- B
          const int gb = (args.mode == kGroupedM) ? ti.g : 0;
          const int kb = (args.mode == kGroupedK) ? ti.k_row0 + kk : kk;
          if (args.b_split == kBDual) {
            // first half of the tile's columns from source 0 (gate), second half from source 1 (value)
            if (!args.b_mn) {
              tma_load_3d(sB, &tmB0, &full_bar[stage], kb, ti.n0, gb);
              tma_load_3d(sB + (BN / 2) * 128, &tmB1, &full_bar[stage], kb, ti.n0, gb);
            } else {
#pragma unroll
              for (int c = 0; c < BN / 64; ++c) {
                const CUtensorMap* mp = (c < BN / 128) ? &tmB0 : &tmB1;
                const int nc = ti.n0 + 64 * (c % (BN / 128));
                tma_load_3d(sB + c * 8192, mp, &full_bar[stage], nc, kb, gb);
              }
            }
          } else {
            const CUtensorMap* mp = &tmB0;
            int nb = ti.n0, kcoord = kb;
            if (args.b_split == kBSplitN) {
              const int src = ti.n0 / args.b_split_size;
              mp = src == 0 ? &tmB0 : (src == 1 ? &tmB1 : &tmB2);
              nb = ti.n0 - src * args.b_split_size;
            } else if (args.b_split == kBSplitK) {
              const int src = kb / args.b_split_size;
              mp = src == 0 ? &tmB0 : (src == 1 ? &tmB1 : &tmB2);
              kcoord = kb - src * args.b_split_size;
            }
            if (!args.b_mn) {
              tma_load_3d(sB, mp, &full_bar[stage], kcoord, nb, gb);
            } else {
#pragma unroll
              for (int c = 0; c < BN / 64; ++c)
                tma_load_3d(sB + c * 8192, mp, &full_bar[stage], nb + 64 * c, kcoord, gb);
            }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < n_total && ok; t += gridDim.x) {
      const Tile ti = get_tile<BN, EPI>(args, tile_start, t);
      if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1u, abort_flag, args.status, kKernelGemm, 200 + acc)) { ok = false; break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
      if (ti.k_chunks == 0) {
        if (lane == 0) mbar_arrive(&tmem_full[acc]);
      }
      for (int kc = 0; kc < ti.k_chunks; ++kc) {
        if (!mbar_wait(&full_bar[stage], phase, abort_flag, args.status, kKernelGemm, 300 + stage)) { ok = false; break; }
        tc_fence_after();
        uint8_t* sA = smem + stage * S::STAGE_BYTES;
        uint8_t* sB = sA + A_STAGE_BYTES;
        if (args.mode == kGroupedK) {
          // Rows past the end of the segment belong to the next expert: zero them in both tiles.
          const int valid = ti.k_rows - kc * BK;
          if (valid < BK) {
            for (int r = valid; r < BK; ++r) {
              for (int c = 0; c < 2; ++c) reinterpret_cast<uint32_t*>(sA + c * 8192 + r * 128)[lane] = 0u;
              for (int c = 0; c < BN / 64; ++c) reinterpret_cast<uint32_t*>(sB + c * 8192 + r * 128)[lane] = 0u;
            }
            fence_proxy_async_smem();
            __syncwarp();
          }
        }
        if (lane == 0) {
          const uint32_t a_addr = smem_u32(sA), b_addr = smem_u32(sB);
#pragma unroll
          for (int ks = 0; ks < BK / 16; ++ks) {
            const uint64_t da = args.a_mn ? smem_desc_sw128(a_addr + ks * 2048, 8192, 1024)
                                          : smem_desc_sw128(a_addr + ks * 32, 16, 1024);
            const uint64_t db = args.b_mn ? smem_desc_sw128(b_addr + ks * 2048, 8192, 1024)
                                          : smem_desc_sw128(b_addr + ks * 32, 16, 1024);
            umma_f16(d_tmem, da, db, idesc, (kc | ks) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (kc == ti.k_chunks - 1) umma_commit(&tmem_full[acc]);
        }
        __syncwarp();
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9)
    // A warp reads the TMEM lanes of its quarter (warp index mod 4); warps 2-5 drain the first
    // half of the tile's columns, warps 6-9 the second half.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    constexpr int SPAN = (EPI == kEpiSwigluFwd ? BN / 2 : BN) / 2;  // columns per warp
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
    for (int t = blockIdx.x; t < n_total && ok; t += gridDim.x) {
      const Tile ti = get_tile<BN, EPI>(args, tile_start, t);
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag, args.status, kKernelGemm, 400 + acc)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + static_cast<uint32_t>(acc * BN) + (static_cast<uint32_t>(quarter * 32) << 16);
      const bool row_ok = row_in_tile < ti.rows_valid;
      const bool have_acc = ti.k_chunks > 0;
      const long long row = static_cast<long long>(ti.m0) + row_in_tile;
      // Staged stores clip at the matrix edge only: inside a grouped problem they are used for
      // 32-row groups that lie entirely in the tile's segment.
      const int warp_rows = max(0, min(32, ti.rows_valid - quarter * 32));
      st.on = args.c_tma != 0 && warp_rows > 0 && (args.mode == kDense || warp_rows == 32);
      st.row0 = ti.m0 + quarter * 32;

      epilogue_rows<BN, EPI>(args, ti, t_addr, row_ok, have_acc, row, c_lo, c_hi, st);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (lane == 0) tma_store_wait_read<0>();  // shared memory stays allocated until the last store has read it
  }

  // ---------------------------------------------------------------------- teardown
  __syncwarp();
  if (*abort_flag != 0u) __nanosleep(200000);  // let copies still in flight land before smem is released
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace gemm
}  // namespace nt
