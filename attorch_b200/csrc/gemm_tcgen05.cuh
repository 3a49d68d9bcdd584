// Persistent, warp-specialised tcgen05 GEMM for sm_100a:
//
//     D[M, N] = A[M, K] * B[K, N]        (fp32 accumulation in tensor memory)
//
// with either operand K-major (reduction dimension contiguous in global memory) or MN-major
// (output dimension contiguous).  The three GEMMs of the fused linear layer map onto it as
//
//     forward   Y  = X  * W      A = X   K-major,   B = W   MN-major   (W is [in, out], out contiguous)
//     backward  dX = dZ * W^T    A = dZ  K-major,   B = W   K-major
//     backward  dW = X^T * dZ    A = X   MN-major,  B = dZ  MN-major
//     skinny    Y^T = W^T * X^T  A = W   MN-major,  B = X   K-major    (swap-AB, stream-K)
//
// which replaces the reference's Triton tile loop (attorch/linear_kernels.py:143-165) and the two
// cuBLAS matmuls of its backward (attorch/linear_layer.py:152-155).
//
// Structure of one CTA (320 threads, one CTA per SM, grid = min(work, #SM)):
//   warp 0      TMA producer: fills a ring of kStages shared-memory stages (A tile + B tile,
//               128-byte swizzle) with cp.async.bulk.tensor, completion on "full" mbarriers.
//   warp 1      MMA issuer: one thread issues tcgen05.mma (128 x BN x 32 bytes of K each) from the
//               shared-memory descriptors into one of two accumulators in tensor memory;
//               tcgen05.commit releases the stage ("empty") and publishes the accumulator.
//   warps 2-9   epilogue: tcgen05.ld the finished accumulator (a warp may read the 32 TMEM lanes of
//               its quarter, warp id mod 4; the two warps of a quarter take alternate 32-column
//               chunks), add bias, store the pre-activation, apply the activation, store the output.
//               The second accumulator lets the epilogue of tile i overlap the main loop of tile
//               i + 1; two warps per scheduler keep its latency below the main loop's.
//
// Work is either whole output tiles (tile-parallel, direct epilogue) or equal contiguous ranges of
// (tile, k-block) units (stream-K, fp32 atomic accumulation into a zeroed workspace that a small
// finishing kernel turns into the output).
//
// With kCtas = 2 two CTAs on the two SMs of a TPC (a cluster of 2) share one 256 x BN tile: each
// loads its own 128 rows of A and its own half of the columns of B, and the leader CTA (cluster
// rank 0) issues tcgen05.mma.cta_group::2, which reads both CTAs' shared memory and writes 128
// accumulator rows into each CTA's tensor memory.  Per SM that halves the B bytes pulled through L2
// and read from shared memory.  Both CTAs' TMA loads complete on the leader's "full" barrier; the
// leader's tcgen05.commit signals "empty" and "accumulator full" in both CTAs; both CTAs' epilogue
// warps arrive on the leader's "accumulator empty" barrier.  No load is multicast.
#pragma once
#include "act_math.cuh"
#include "common.cuh"
#include "ptx.cuh"

namespace ab200 {

struct GemmArgs {
  int M, N, K;            // output rows, output columns, reduction length
  int tiles_m, tiles_n;   // ceil(M / 128), ceil(N / BN)
  int group_m;            // row-blocks per rasterisation group
  int k_blocks;           // ceil(K / elements per stage)
  int stream_k;           // 0: whole tiles; 1: equal (tile, k-block) shares + atomics; 2: hybrid;
                          // 3: whole tiles, those of the partial last round as two half-width tiles
  int dp_tiles;           // modes 2, 3: tiles computed whole (a multiple of the worker count)
  uint32_t idesc;         // tcgen05 instruction descriptor (operand format, majorness, 128 x BN)
  // Direct epilogue
  void* out;              // [M, N], row pitch ld_out elements
  long long ld_out;
  int out_dtype;
  void* aux;              // optional second output written before the activation (pre-activation)
  long long ld_aux;
  const void* bias;       // optional [N]
  int bias_dtype;
  int act;
  float act_param;
  const void* residual;   // optional [M, N] in the output dtype, added after the activation
  long long ld_res;
  // Stream-K epilogue
  float* partial;         // fp32; mode 1: zero on entry, [M, N] (pitch ld_partial) or, if transposed,
                          // [N, M]; mode 2: 2 * workers dense TILE_M x BN slots, written through a map
  long long ld_partial;
  int partial_transposed;
  int* status;            // device word; a bounded wait that runs out stores a DeviceStatus here
  int save_grad;          // aux receives act'(Z) instead of Z (see actm::fwd_grad)
  int grad_dtype;         // element type act'(Z) is stored in (2 bytes if out_dtype is; see api.cu)
  int tma_store;          // bit 0: `out` goes through shared memory and a TMA store; bit 1: `aux` too
  // Gated linear unit in the epilogue (forward only, B MN-major, whole tiles): B is [K, 2 * gate_cols],
  // a tile multiplies BN / 2 columns of the first half and the matching BN / 2 columns of the second,
  // aux receives both pre-activation halves ([M, 2 * gate_cols]) and out = x1 * act(x2) ([M, gate_cols]).
  // N is then gate_cols; 0 switches it off.
  int gate_cols;
};

template <int BN_, int ELT_, bool A_MN_, bool B_MN_, int CTAS_ = 1>
struct GemmCfg {
  static constexpr int CTAS = CTAS_;             // CTAs sharing one tile (1, or 2 with cta_group::2)
  static constexpr int BM = 128;                 // accumulator rows per CTA
  static constexpr int TILE_M = BM * CTAS;       // output rows per tile
  static constexpr int BN = BN_;
  static constexpr int BN_CTA = BN_ / CTAS_;     // columns of B each CTA loads
  static constexpr int ELT = ELT_;               // bytes per operand element (2: f16/bf16, 4: tf32)
  static constexpr bool A_MN = A_MN_;
  static constexpr bool B_MN = B_MN_;
  static constexpr int BKE = 128 / ELT;          // K elements per stage (one 128-byte swizzle row)
  static constexpr int UMMA_K = 32 / ELT;        // K elements per tcgen05.mma
  static constexpr int A_BYTES = BM * 128;
  static constexpr int B_BYTES = BN_CTA * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int kMaxSmem = 227 * 1024;
  static constexpr int kBarrierBytes = 512;
  static constexpr int kEpilogueWarps = 8;
  // Each epilogue warp stages one 32 x 32 chunk (up to 4 bytes per element) for its TMA stores.
  static constexpr int kStageOutBytes = 32 * 32 * 4;
  static constexpr int kStoreBytes = kEpilogueWarps * kStageOutBytes;
  static constexpr int kStagesFit = (kMaxSmem - 1024 - kBarrierBytes - kStoreBytes) / STAGE_BYTES;
  static constexpr int STAGES = kStagesFit > 8 ? 8 : kStagesFit;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + kStoreBytes + 1024 + kBarrierBytes;
  static constexpr int TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;   // power of two for BN in {16..256}
  static constexpr int MN_ATOM = 128 / ELT;      // elements in one 128-byte row of an MN-major tile
  // A K-major B tile is fetched as two boxes of half its rows, so that a half-width unit (see
  // SegmentIter, mode 3) fetches exactly the rows it multiplies.
  static constexpr int B_BOX_ROWS = BN_CTA >= 16 ? BN_CTA / 2 : BN_CTA;
  // Can a tile be computed as two units of BN / 2 columns?  Each CTA's share of a unit must be whole
  // TMA boxes: half a K-major tile, or whole 128-byte column blocks of an MN-major one.
  static constexpr bool kHalfUnits = BN_ >= 64 && (B_MN_ ? (BN_CTA / 2) % (128 / ELT_) == 0 : BN_CTA >= 16);
  static constexpr int MN_BOX_BYTES = BKE * 128; // one TMA box of an MN-major tile
  // MN-major tiles of 4-byte elements use the 128-byte swizzle with 32-byte units, whose pattern
  // repeats every 4 rows of K; everything else the ordinary one (16-byte units, 8 rows).
  static constexpr bool MN_BASE32 = (ELT == 4);
  static constexpr uint32_t MN_LAYOUT = MN_BASE32 ? ptx::kLayoutSw128Base32 : ptx::kLayoutSw128;
  static constexpr uint32_t MN_SBO = MN_BASE32 ? 512 : 1024;
  static constexpr int kThreads = 32 * (2 + kEpilogueWarps);
  static_assert(BN % 32 == 0 && BN >= 32 && BN <= 256, "BN must be 32, 64, 128 or 256");
  static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0, "TMEM allocation must be a power of two");
  static_assert(!B_MN_ || BN_CTA % (128 / ELT_) == 0, "an MN-major B tile is made of 128-byte wide boxes");
  static_assert(CTAS_ == 1 || CTAS_ == 2, "one CTA or a pair");
};

// Most workers whose pieces the finishing pass of the hybrid schedule can sum for one tile (it keeps
// one slot index per worker in shared memory); launches with more workers use whole tiles instead.
// B200 has 148 SMs.
constexpr int kMaxTailPieces = 160;

struct Segment {
  int m_blk, n_blk;
  int n_off, n_cols;  // columns [n_off, n_off + n_cols) of the tile: all BN of them, or one half
  int kb0, kb1;     // k-block range [kb0, kb1)
  int partial;      // 1: add the result to the fp32 partial sums; 0: whole tile, fused epilogue
  int sk_index;     // hybrid mode: slot of this worker's partial tile (2 * worker + 0 or 1)
};

// Tile index -> (row block, column block).  Grouped rasterisation: group_m row blocks at a time,
// row-block index fastest.
__host__ __device__ __forceinline__ void tile_to_blocks(int t, int tiles_m, int tiles_n, int group_m,
                                                        int& m_blk, int& n_blk) {
  const int per_group = group_m * tiles_n;
  const int g = t / per_group;
  const int first_m = g * group_m;
  const int gsz = (tiles_m - first_m < group_m) ? tiles_m - first_m : group_m;
  const int r = t - g * per_group;
  m_blk = first_m + r % gsz;
  n_blk = r / gsz;
}

// Every role of a CTA walks the same sequence of segments, computed from its worker index alone.
//   stream_k = 0  whole tiles: worker, worker + workers, ...
//   stream_k = 1  all (tile, k-block) units in equal contiguous shares
//   stream_k = 2  hybrid: the first dp_tiles tiles whole, as in mode 0 (dp_tiles is a multiple of
//                 the worker count, so these are full rounds); the (tile, k-block) units of the
//                 remaining tiles in equal shares, which spreads a partial last round over all SMs.
//                 A share is shorter than one tile's reduction, so it touches at most two tiles;
//                 each piece is written, not added, to the worker's own slot (2 * worker, then
//                 2 * worker + 1) and a finishing kernel sums the slots of a tile in worker order:
//                 no atomics, no clearing, bit-repeatable.
//   stream_k = 3  the first dp_tiles tiles whole, as in mode 0; each remaining tile as two units of
//                 BN / 2 columns (unit h = column half h % 2 of tile dp_tiles + h / 2), handed out
//                 like tiles.  A last round that would occupy at most half of the workers then takes
//                 half as long, every unit still ends in the fused epilogue, and the epilogue that
//                 nothing overlaps - the one after a worker's last main loop - is that of half a tile.
struct SegmentIter {
  long long unit, unit_end;   // position in the shared-out (tile, k-block) units
  int tile, tile_end;         // next whole tile
  int stride;                 // number of workers (CTAs, or CTA pairs)
  int first_shared;           // first tile whose units are shared out
  int slot;                   // hybrid: next partial-tile slot of this worker
  // worker / workers: index and count of the CTAs (or CTA pairs) that share the work.
  __device__ __forceinline__ SegmentIter(const GemmArgs& a, int worker, int workers) {
    const int tiles = a.tiles_m * a.tiles_n;
    stride = workers;
    tile = worker;
    slot = 2 * worker;
    tile_end = a.stream_k == 0 ? tiles : (a.stream_k >= 2 ? a.dp_tiles : 0);
    first_shared = a.stream_k == 0 ? tiles : (a.stream_k >= 2 ? a.dp_tiles : 0);
    if (a.stream_k == 3) {
      unit = worker;                                   // half-width units, round robin
      unit_end = 2ll * (tiles - first_shared);
    } else {
      const long long total = static_cast<long long>(tiles - first_shared) * a.k_blocks;
      unit = total * worker / workers;
      unit_end = total * (worker + 1) / workers;
    }
  }
  __device__ __forceinline__ bool next(const GemmArgs& a, Segment& s, int bn) {
    int t;
    s.n_off = 0;
    s.n_cols = bn;
    if (tile < tile_end) {
      t = tile;
      tile += stride;
      s.kb0 = 0;
      s.kb1 = a.k_blocks;
      s.partial = 0;
      s.sk_index = 0;
    } else if (a.stream_k == 3) {
      // Half-width units; one whose columns all lie beyond N (second half of a ragged last column
      // block) is skipped - by every role alike, since all walk this same sequence.
      for (;;) {
        if (unit >= unit_end) return false;
        t = first_shared + static_cast<int>(unit >> 1);
        s.n_off = static_cast<int>(unit & 1) * (bn / 2);
        unit += stride;
        tile_to_blocks(t, a.tiles_m, a.tiles_n, a.group_m, s.m_blk, s.n_blk);
        if (s.n_blk * bn + s.n_off < a.N) break;
      }
      s.n_cols = bn / 2;
      s.kb0 = 0;
      s.kb1 = a.k_blocks;
      s.partial = 0;
      s.sk_index = 0;
    } else {
      if (unit >= unit_end) return false;
      const int ts = static_cast<int>(unit / a.k_blocks);
      t = first_shared + ts;
      s.kb0 = static_cast<int>(unit - static_cast<long long>(ts) * a.k_blocks);
      const long long left = unit_end - unit;
      s.kb1 = (a.k_blocks - s.kb0 < left) ? a.k_blocks : s.kb0 + static_cast<int>(left);
      unit += s.kb1 - s.kb0;
      s.partial = 1;
      s.sk_index = slot++;
    }
    tile_to_blocks(t, a.tiles_m, a.tiles_n, a.group_m, s.m_blk, s.n_blk);
    return true;
  }
};

// Stores up to 32 consecutive columns of one output row.
__device__ __forceinline__ void store_row_chunk(void* base, int dt, long long offset,
                                                const float (&v)[32], int valid) {
  if (dt == DT_F32) {
    float* p = static_cast<float*>(base) + offset;
    if (valid == 32 && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        reinterpret_cast<float4*>(p)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i < valid) p[i] = v[i];
    }
  } else {
    uint16_t* p = static_cast<uint16_t*>(base) + offset;
    if (valid == 32 && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint4 q;
        q.x = pack2(v[8 * i + 0], v[8 * i + 1], dt);
        q.y = pack2(v[8 * i + 2], v[8 * i + 3], dt);
        q.z = pack2(v[8 * i + 4], v[8 * i + 5], dt);
        q.w = pack2(v[8 * i + 6], v[8 * i + 7], dt);
        reinterpret_cast<uint4*>(p)[i] = q;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i < valid) store_from_f32(p, dt, i, v[i]);
    }
  }
}

// Writes this lane's row of a 32 x 32 chunk (lane = row, v = its 32 columns, rounded to dt) into the
// warp's staging buffer in the layout a swizzled TMA store expects: rows of 64 bytes with the
// 64-byte swizzle for 2-byte elements, rows of 128 bytes with the 128-byte swizzle for fp32 (16-byte
// unit j of row r sits at unit j ^ ((r >> 1) & 3), resp. j ^ (r & 7)); conflict-free per quarter warp.
__device__ __forceinline__ void stage_row_chunk(uint32_t buf, int lane, int dt, const float (&v)[32]) {
  if (dt == DT_F32) {
    const uint32_t row = buf + lane * 128;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      ptx::st_shared_v4(row + ((j ^ (lane & 7)) << 4), __float_as_uint(v[4 * j]), __float_as_uint(v[4 * j + 1]),
                        __float_as_uint(v[4 * j + 2]), __float_as_uint(v[4 * j + 3]));
  } else {
    const uint32_t row = buf + lane * 64;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      ptx::st_shared_v4(row + ((j ^ ((lane >> 1) & 3)) << 4), pack2(v[8 * j], v[8 * j + 1], dt),
                        pack2(v[8 * j + 2], v[8 * j + 3], dt), pack2(v[8 * j + 4], v[8 * j + 5], dt),
                        pack2(v[8 * j + 6], v[8 * j + 7], dt));
  }
}

// v[i] += bias[col0 + i] for the valid columns of a 32-column chunk (same addresses in every lane:
// the loads are warp-wide broadcasts, 16 bytes at a time when the chunk is whole and aligned).
// A bias wider than the output type is first rounded to it (round_dt), as the reference does when
// the output is 16-bit (attorch/linear_kernels.py:171-172).
__device__ __forceinline__ void add_bias_chunk(float (&v)[32], const void* bias, int dt, int col0,
                                               int valid, int round_dt) {
  const int elt = dt == DT_F32 ? 4 : 2;
  const char* p = static_cast<const char*>(bias) + static_cast<long long>(col0) * elt;
  if (valid == 32 && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
    if (dt == DT_F32) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float4 b = __ldg(reinterpret_cast<const float4*>(p) + i);
        round_through2(b.x, b.y, round_dt);
        round_through2(b.z, b.w, round_dt);
        const float2 lo = actm::add2(make_float2(v[4 * i], v[4 * i + 1]), make_float2(b.x, b.y));
        const float2 hi = actm::add2(make_float2(v[4 * i + 2], v[4 * i + 3]), make_float2(b.z, b.w));
        v[4 * i] = lo.x; v[4 * i + 1] = lo.y; v[4 * i + 2] = hi.x; v[4 * i + 3] = hi.y;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 b = __ldg(reinterpret_cast<const uint4*>(p) + i);
        const uint32_t w[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float lo, hi;
          if (dt == DT_F16) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
            lo = f.x; hi = f.y;
          } else {
            lo = __uint_as_float(w[j] << 16);
            hi = __uint_as_float(w[j] & 0xFFFF0000u);
          }
          v[8 * i + 2 * j] += lo;
          v[8 * i + 2 * j + 1] += hi;
        }
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < valid) v[i] += round_through(load_as_f32(bias, dt, col0 + i), round_dt);
  }
}

// v[i] += residual[row, col0 + i] for the valid columns of a 32-column chunk of one row (16 bytes at a
// time when the chunk is whole and aligned).
__device__ __forceinline__ void add_residual_chunk(float (&v)[32], const void* residual, int dt, long long offset,
                                                   int valid) {
  const int elt = dt == DT_F32 ? 4 : 2;
  const char* p = static_cast<const char*>(residual) + offset * elt;
  if (valid == 32 && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
    if (dt == DT_F32) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4 r = __ldg(reinterpret_cast<const float4*>(p) + i);
        v[4 * i] += r.x; v[4 * i + 1] += r.y; v[4 * i + 2] += r.z; v[4 * i + 3] += r.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 r = __ldg(reinterpret_cast<const uint4*>(p) + i);
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float lo, hi;
          if (dt == DT_F16) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
            lo = f.x; hi = f.y;
          } else {
            lo = __uint_as_float(w[j] << 16);
            hi = __uint_as_float(w[j] & 0xFFFF0000u);
          }
          v[8 * i + 2 * j] += lo;
          v[8 * i + 2 * j + 1] += hi;
        }
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < valid) v[i] += load_as_f32(residual, dt, offset + i);
  }
}

template <class Cfg>
__global__ void __launch_bounds__(Cfg::kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a,
                    const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_out,
                    const __grid_constant__ CUtensorMap tmap_aux,
                    const __grid_constant__ CUtensorMap tmap_partial, const GemmArgs args) {
  constexpr int BM = Cfg::BM, BN = Cfg::BN, BKE = Cfg::BKE, STAGES = Cfg::STAGES;
  constexpr int CTAS = Cfg::CTAS;
  constexpr bool kTf32 = (Cfg::ELT == 4);
  constexpr bool kPair = (CTAS == 2);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;
  uint8_t* smem = smem_raw + pad;              // 1024-byte aligned: required by the 128-byte swizzle
  const uint32_t smem_base = raw_addr + pad;
  const uint32_t store_base = smem_base + STAGES * Cfg::STAGE_BYTES;   // 1024-byte aligned
  uint8_t* bar_region = smem + STAGES * Cfg::STAGE_BYTES + Cfg::kStoreBytes;
  const uint32_t bar_base = store_base + Cfg::kStoreBytes;
  // Barrier layout (8 bytes each): full[STAGES], empty[STAGES], acc_full[2], acc_empty[2].
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto acc_full_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
  auto acc_empty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_region + 8 * (2 * STAGES + 4));
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // Rank of this CTA in its pair (0 = leader, which issues the MMAs) and the pair's place among
  // the workers that share the tiles.
  const uint32_t cta = kPair ? ptx::cluster_ctarank() : 0u;
  const int worker = static_cast<int>(blockIdx.x) / CTAS;
  const int workers = static_cast<int>(gridDim.x) / CTAS;

  if (warp == 0 && lane == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(full_bar(s), 1);        // the leader's arrive.expect_tx
      ptx::mbar_init(empty_bar(s), 1);       // one tcgen05.commit
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(acc_full_bar(b), 1);    // one tcgen05.commit
      ptx::mbar_init(acc_empty_bar(b), Cfg::kEpilogueWarps * CTAS);   // one arrival per epilogue warp
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tmap(&tmap_a);
    ptx::prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    ptx::tmem_alloc<CTAS>(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), Cfg::TMEM_COLS);
    ptx::tmem_relinquish<CTAS>();
  }
  ptx::tc_fence_before_sync();
  if constexpr (kPair) {
    // The peer's barriers must be initialised before anything here signals them.
    ptx::cluster_arrive();
    ptx::cluster_wait();
  } else {
    __syncthreads();
  }
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // A bounded wait that also gives up as soon as another role of this CTA has given up.
  auto wait = [&](uint32_t bar, uint32_t parity, int code) -> bool {
    uint32_t spins = 0;
    uint64_t t0 = 0;
    while (!(kPair ? ptx::mbar_try_wait_cluster(bar, parity) : ptx::mbar_try_wait(bar, parity))) {
      if ((++spins & 0x3FFu) == 0) {
        if (*abort_flag) return false;
        const uint64_t now = ptx::globaltimer_ns();
        if (t0 == 0) {
          t0 = now;
        } else if (now - t0 > ptx::kWaitLimitNs) {
          *abort_flag = 1;
          atomicCAS(args.status, 0, code);
          return false;
        }
      }
    }
    return true;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      SegmentIter it(args, worker, workers);
      Segment seg;
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      while (ok && it.next(args, seg, BN)) {
        const int m0 = seg.m_blk * Cfg::TILE_M + static_cast<int>(cta) * BM;      // this CTA's rows of A
        // This CTA's columns of B: BN_CTA of them, or half as many for a half-width unit, which
        // fetches (and expects the bytes of) only those.
        const int b_cols = seg.n_cols / CTAS;
        const int n0 = seg.n_blk * BN + seg.n_off + static_cast<int>(cta) * b_cols;
        const uint32_t stage_tx = Cfg::A_BYTES + static_cast<uint32_t>(b_cols) * 128u;
        for (int kb = seg.kb0; kb < seg.kb1; ++kb) {
          if (!wait(empty_bar(s), ph ^ 1u, DEV_TIMEOUT_PRODUCER)) { ok = false; break; }
          // The pair's loads all complete on the leader's barrier, which expects both CTAs' bytes.
          uint32_t full = full_bar(s);
          if constexpr (kPair) {
            if (cta == 0) ptx::mbar_arrive_expect_tx(full, stage_tx * CTAS);
            full = ptx::map_to_cta(full, 0);
          } else {
            ptx::mbar_arrive_expect_tx(full, stage_tx);
          }
          const uint32_t a_dst = smem_base + s * Cfg::STAGE_BYTES;
          const uint32_t b_dst = a_dst + Cfg::A_BYTES;
          const int k0 = kb * BKE;
          if constexpr (Cfg::A_MN) {
#pragma unroll
            for (int j = 0; j < BM / Cfg::MN_ATOM; ++j)
              ptx::tma_load_2d<kPair>(a_dst + j * Cfg::MN_BOX_BYTES, &tmap_a, full, m0 + j * Cfg::MN_ATOM, k0);
          } else {
            ptx::tma_load_2d<kPair>(a_dst, &tmap_a, full, k0, m0);
          }
          if constexpr (Cfg::B_MN) {
#pragma unroll
            for (int j = 0; j < Cfg::BN_CTA / Cfg::MN_ATOM; ++j)
              if (j * Cfg::MN_ATOM < b_cols) {
                int col = n0 + j * Cfg::MN_ATOM;
                if (args.gate_cols) {
                  // Column t of the tile: first half of the gated pair for t < BN / 2, else second half.
                  const int t = static_cast<int>(cta) * b_cols + j * Cfg::MN_ATOM;
                  col = seg.n_blk * (BN / 2) + (t < BN / 2 ? t : args.gate_cols + t - BN / 2);
                }
                ptx::tma_load_2d<kPair>(b_dst + j * Cfg::MN_BOX_BYTES, &tmap_b, full, col, k0);
              }
          } else {
#pragma unroll
            for (int j = 0; j < Cfg::BN_CTA / Cfg::B_BOX_ROWS; ++j)
              if (j * Cfg::B_BOX_ROWS < b_cols)
                ptx::tma_load_2d<kPair>(b_dst + j * Cfg::B_BOX_ROWS * 128, &tmap_b, full, k0, n0 + j * Cfg::B_BOX_ROWS);
          }
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && cta == 0) {
      SegmentIter it(args, worker, workers);
      Segment seg;
      int s = 0;
      uint32_t ph = 0;
      uint32_t n_acc = 0;
      bool ok = true;
      while (ok && it.next(args, seg, BN)) {
        const uint32_t b = n_acc & 1u;
        const uint32_t acc_ph = (n_acc >> 1) & 1u;
        if (!wait(acc_empty_bar(b), acc_ph ^ 1u, DEV_TIMEOUT_MMA)) { ok = false; break; }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + b * BN;
        // Instruction descriptor with this unit's N (bits 17-22 hold N / 8).
        const uint32_t idesc = args.idesc - (static_cast<uint32_t>((BN - seg.n_cols) >> 3) << 17);
        for (int kb = seg.kb0; kb < seg.kb1; ++kb) {
          if (!wait(full_bar(s), ph, DEV_TIMEOUT_MMA)) { ok = false; break; }
          ptx::tc_fence_after_sync();
          const uint32_t a_addr = smem_base + s * Cfg::STAGE_BYTES;
          const uint32_t b_addr = a_addr + Cfg::A_BYTES;
#pragma unroll
          for (int k = 0; k < BKE / Cfg::UMMA_K; ++k) {
            // K-major: the next 32 bytes of every 128-byte row.  MN-major: the next UMMA_K rows.
            const uint64_t a_desc =
                Cfg::A_MN ? ptx::make_smem_desc(a_addr + k * Cfg::UMMA_K * 128, Cfg::MN_BOX_BYTES,
                                                Cfg::MN_SBO, Cfg::MN_LAYOUT)
                          : ptx::make_smem_desc(a_addr + k * 32, 16, 1024);
            const uint64_t b_desc =
                Cfg::B_MN ? ptx::make_smem_desc(b_addr + k * Cfg::UMMA_K * 128, Cfg::MN_BOX_BYTES,
                                                Cfg::MN_SBO, Cfg::MN_LAYOUT)
                          : ptx::make_smem_desc(b_addr + k * 32, 16, 1024);
            ptx::umma<CTAS, kTf32>(d_tmem, a_desc, b_desc, idesc, (kb > seg.kb0 || k > 0) ? 1u : 0u);
          }
          // The stage is reusable (in both CTAs) once these MMAs have read it.
          if constexpr (kPair) ptx::umma_commit_pair(empty_bar(s), 3);
          else ptx::umma_commit(empty_bar(s));
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
        if (!ok) break;
        // Accumulator complete (in both CTAs' tensor memory).
        if constexpr (kPair) ptx::umma_commit_pair(acc_full_bar(b), 3);
        else ptx::umma_commit(acc_full_bar(b));
        ++n_acc;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9)
    const int q = warp & 3;                    // TMEM lane quarter this warp may access
    const int half = (warp - 2) >> 2;          // which of the quarter's two warps: chunks half, half + 2, ...
    const uint32_t stage_buf = store_base + (warp - 2) * Cfg::kStageOutBytes;
    SegmentIter it(args, worker, workers);
    Segment seg;
    uint32_t n_acc = 0;
    bool ok = true;
    while (ok && it.next(args, seg, BN)) {
      const uint32_t b = n_acc & 1u;
      const uint32_t acc_ph = (n_acc >> 1) & 1u;
      if (!wait(acc_full_bar(b), acc_ph, DEV_TIMEOUT_EPILOGUE)) { ok = false; break; }
      ptx::tc_fence_after_sync();
      const int row = seg.m_blk * Cfg::TILE_M + static_cast<int>(cta) * BM + q * 32 + lane;
      const bool row_ok = row < args.M;
      if (args.gate_cols) {
        // Gated linear unit: chunk c of the first half pairs with chunk c of the second half.
        constexpr int HB = BN / 2;
        const int row0 = seg.m_blk * Cfg::TILE_M + static_cast<int>(cta) * BM + q * 32;
        const uint32_t t_acc = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + b * BN;
        auto emit_at = [&](const CUtensorMap* map, void* base, long long ld, bool by_tma, const float (&w)[32],
                           int col, int valid) {
          if (by_tma) {
            if (lane == 0) ptx::tma_store_wait_read();
            __syncwarp();
            stage_row_chunk(stage_buf, lane, args.out_dtype, w);
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0 && row0 < args.M) {
              ptx::tma_store_2d(map, stage_buf, col, row0);
              ptx::tma_store_commit();
            }
          } else if (row_ok) {
            store_row_chunk(base, args.out_dtype, static_cast<long long>(row) * ld + col, w, valid);
          }
        };
#pragma unroll 1
        for (int c = half; c < HB / 32; c += Cfg::kEpilogueWarps / 4) {
          const int col0 = seg.n_blk * HB + c * 32;           // column within each half
          if (col0 >= args.gate_cols) break;                  // warp-uniform
          const int valid = (args.gate_cols - col0 < 32) ? args.gate_cols - col0 : 32;
          uint32_t r1[32], r2[32];
          ptx::tmem_ld_32x32(t_acc + c * 32, r1);
          ptx::tmem_ld_32x32(t_acc + HB + c * 32, r2);
          ptx::tmem_ld_wait();
          float x1[32], x2[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            x1[i] = __uint_as_float(r1[i]);
            x2[i] = __uint_as_float(r2[i]);
          }
          if (args.bias != nullptr) {
            add_bias_chunk(x1, args.bias, args.bias_dtype, col0, valid, args.out_dtype);
            add_bias_chunk(x2, args.bias, args.bias_dtype, args.gate_cols + col0, valid, args.out_dtype);
          }
          if (args.aux != nullptr) {
            // tmap_partial covers the first half only ([M, gate_cols]), so that a ragged last chunk of
            // it is clipped instead of spilling into the second half's columns.
            emit_at(&tmap_partial, args.aux, args.ld_aux, (args.tma_store & 2) != 0, x1, col0, valid);
            emit_at(&tmap_aux, args.aux, args.ld_aux, (args.tma_store & 2) != 0, x2, args.gate_cols + col0, valid);
          }
          // The unit multiplies the halves as they are stored (rounded to the output type), which is
          // what a separate gated-linear-unit pass over the stored pre-activation reads
          // (attorch/glu_kernels.py:45-52).
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            x1[i] = round_through(x1[i], args.out_dtype);
            x2[i] = round_through(x2[i], args.out_dtype);
          }
          act_fwd_inplace(x2, args.act, args.act_param);
#pragma unroll
          for (int i = 0; i < 32; ++i) x1[i] *= x2[i];
          emit_at(&tmap_out, args.out, args.ld_out, (args.tma_store & 1) != 0, x1, col0, valid);
        }
      } else {
#pragma unroll 1
      for (int c = half; c < seg.n_cols / 32; c += Cfg::kEpilogueWarps / 4) {
        const int col0 = seg.n_blk * BN + seg.n_off + c * 32;
        if (col0 >= args.N) break;             // warp-uniform
        uint32_t r[32];
        ptx::tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + b * BN + c * 32, r);
        ptx::tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
        const int valid = (args.N - col0 < 32) ? args.N - col0 : 32;
        if (seg.partial) {
          if (args.stream_k == 2) {
            // This worker's own slot: a plain fp32 TMA store of the chunk.
            if (lane == 0) ptx::tma_store_wait_read();
            __syncwarp();
            stage_row_chunk(stage_buf, lane, DT_F32, v);
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              ptx::tma_store_2d(&tmap_partial, stage_buf, c * 32,
                                seg.sk_index * Cfg::TILE_M + static_cast<int>(cta) * BM + q * 32);
              ptx::tma_store_commit();
            }
          } else if (row_ok) {
            if (args.partial_transposed) {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (i < valid) atomicAdd(args.partial + static_cast<long long>(col0 + i) * args.ld_partial + row, v[i]);
            } else {
              float* p = args.partial + static_cast<long long>(row) * args.ld_partial + col0;
              if (valid == 32 && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  ptx::red_add_v4_f32(p + 4 * i, v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
              } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                  if (i < valid) atomicAdd(p + i, v[i]);
              }
            }
          }
        } else {
          const int row0 = seg.m_blk * Cfg::TILE_M + static_cast<int>(cta) * BM + q * 32;   // chunk's first row
          // The fused epilogue of one chunk.  kOdt / kGdt fix the output type and the type the saved
          // derivative is stored in at compile time (-1: read them from the arguments): with the types
          // known the conversions and packings are single instructions instead of selections between
          // the variants, which on the forward pass with bias, gelu and a saved derivative is 5 us of 217.
          auto fused = [&]<int kOdt, int kGdt>() {
            const int odt = kOdt >= 0 ? kOdt : args.out_dtype;
            const int gdt = kGdt >= 0 ? kGdt : args.grad_dtype;
            if (args.bias != nullptr) add_bias_chunk(v, args.bias, args.bias_dtype, col0, valid, odt);
            // Writes one 32 x 32 chunk of an output: through the warp's staging buffer and a TMA
            // store, or straight from registers where TMA cannot address the output.
            auto emit = [&](const CUtensorMap* map, void* base, long long ld, bool by_tma, const float (&w)[32], int dt) {
              if (by_tma) {
                // One staging buffer per warp: the previous store must have read it out first.
                if (lane == 0) ptx::tma_store_wait_read();
                __syncwarp();
                stage_row_chunk(stage_buf, lane, dt, w);
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0 && row0 < args.M) {
                  ptx::tma_store_2d(map, stage_buf, col0, row0);
                  ptx::tma_store_commit();
                }
              } else if (row_ok) {
                store_row_chunk(base, dt, static_cast<long long>(row) * ld + col0, w, valid);
              }
            };
            if (args.aux != nullptr && args.save_grad) {
              // Save act'(Z) instead of Z: backward then needs one multiply per element.
              float zr[32], g[32];
#pragma unroll
              for (int i = 0; i < 32; i += 2) {
                zr[i] = v[i];
                zr[i + 1] = v[i + 1];
                round_through2(zr[i], zr[i + 1], odt);
              }
              act_fwd_grad(v, zr, g, args.act, args.act_param);
              emit(&tmap_aux, args.aux, args.ld_aux, (args.tma_store & 2) != 0, g, gdt);
            } else {
              if (args.aux != nullptr) emit(&tmap_aux, args.aux, args.ld_aux, (args.tma_store & 2) != 0, v, odt);
              act_fwd_inplace(v, args.act, args.act_param);
            }
            if (args.residual != nullptr && row_ok)
              add_residual_chunk(v, args.residual, odt, static_cast<long long>(row) * args.ld_res + col0, valid);
            emit(&tmap_out, args.out, args.ld_out, (args.tma_store & 1) != 0, v, odt);
          };
          if (args.out_dtype == DT_BF16 && args.grad_dtype == DT_F16) fused.template operator()<DT_BF16, DT_F16>();
          else if (args.out_dtype == DT_BF16 && args.grad_dtype == DT_BF16) fused.template operator()<DT_BF16, DT_BF16>();
          else fused.template operator()<-1, -1>();
        }
      }
      }
      // This warp has read its share of the accumulator: tell the (leader's) MMA issuer.
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if constexpr (kPair) ptx::mbar_arrive_cluster(acc_empty_bar(b), 0);
        else ptx::mbar_arrive(acc_empty_bar(b));
      }
      ++n_acc;
    }
    // Shared memory must outlive the TMA stores that read it.
    if (lane == 0) ptx::tma_store_wait_all();
  }

  ptx::tc_fence_before_sync();
  if constexpr (kPair) {
    // Neither CTA may free tensor memory or exit while the other can still signal its barriers
    // or while the leader's MMAs still write the peer's accumulators.
    ptx::cluster_arrive();
    ptx::cluster_wait();
  } else {
    __syncthreads();
  }
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc<CTAS>(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace ab200
