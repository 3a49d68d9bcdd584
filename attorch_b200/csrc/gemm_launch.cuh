// Host side of the tcgen05 GEMM: TMA tensor-map construction and the launch of one kernel
// configuration.  The configurations are instantiated in gemm_inst_*.cu, one translation unit per
// (element size, operand majorness) so that they compile in parallel; api.cu picks one through
// launch_tc().
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "common.cuh"
#include "gemm_tcgen05.cuh"

namespace ab200 {

// One GEMM for the tensor-core kernel: operands with their majorness and the pitch (in elements)
// of their strided dimension, the element type, and GemmArgs with M, N, K and the epilogue filled in.
struct TcProblem {
  const void* a; bool a_mn; long long a_pitch;
  const void* b; bool b_mn; long long b_pitch;
  int op_dtype;
  bool allow_pair;   // may run as CTA pairs (cta_group::2) where a configuration for it exists
  bool allow_tma_store;   // the epilogue may write its outputs with TMA stores
  // A partial last round that would keep at most half of the workers busy may run as half-width tiles.
  bool allow_split_tail;
  // SMs this launch leaves free for work that runs beside it (a collective); 0 = none.
  int reserve_sms;
  // Optional scratch for sharing out a partial last round of tiles (hybrid scheduling).
  void* tail_workspace;
  long long tail_workspace_bytes;
  GemmArgs g;
};

// Number of SMs of the current device (148 if it cannot be queried).
int sm_count();

// Row blocks (of 128 rows) per rasterisation group: 4 unless AB200_GROUP_M overrides it (a sweep of
// 2 ... 64 on B200 moved the 8192 x 4096 x 4096 GEMMs by 2 % at most; 2 and 4 were the fastest).
int raster_group_m();

// Upper bound on the CTAs a GEMM launch may use (0 = every SM).  A persistent GEMM that takes every
// SM leaves none for a collective running beside it; a caller that overlaps the two lowers this.
int gemm_cta_limit();
void set_gemm_cta_limit(int ctas);

// Work decomposition (GemmArgs::stream_k) of the last tensor-core GEMM launched from this host thread.
int last_schedule();
void set_last_schedule(int mode);

// AB200_TAIL_MODE (read at every launch): unset / 0 = a last round of tiles that fills at most half of
// the workers runs as half-width units (see launch_cfg); 1 = whole tiles only; 2 = a partial last round
// is shared out over all workers instead (fp32 pieces summed by a finishing kernel) where a workspace
// allows it; 3 = half-width units for every last round.
int tail_mode_override();

// Finishing pass of the hybrid schedule (defined next to the kernel, in api.cu): shared-out tiles
// [first_tile, first_tile + count) of the launch described by g, tile_m x bn each.
int launch_hybrid_finish(const GemmArgs& g, int first_tile, int count, int workers, int tile_m, int bn,
                         cudaStream_t stream);

// Launches p with a BN-wide tile on the kernel family given by p.a_mn / p.b_mn / p.op_dtype.
int launch_tc(const TcProblem& p, int bn, cudaStream_t stream);

// Per-family launchers, defined in gemm_inst_*.cu.  Suffix: element bytes, then the majorness of
// A and B (k = K-major, m = MN-major).
int launch_tc_2_km(const TcProblem& p, int bn, cudaStream_t stream);
int launch_tc_2_kk(const TcProblem& p, int bn, cudaStream_t stream);
int launch_tc_2_mm(const TcProblem& p, int bn, cudaStream_t stream);
int launch_tc_2_mk(const TcProblem& p, int bn, cudaStream_t stream);
int launch_tc_4_km(const TcProblem& p, int bn, cudaStream_t stream);
int launch_tc_4_kk(const TcProblem& p, int bn, cudaStream_t stream);
int launch_tc_4_mm(const TcProblem& p, int bn, cudaStream_t stream);
int launch_tc_4_mk(const TcProblem& p, int bn, cudaStream_t stream);

// 2-D map over a row-major matrix: `inner` contiguous elements per row, `outer` rows, row pitch in
// bytes; box = box_inner x box_outer elements; 128-byte swizzle (of 32-byte units if `atom32`, the
// layout MN-major tf32 operands need); out-of-range elements read as zero.
int encode_2d(CUtensorMap* map, int dtype, const void* base, uint64_t inner, uint64_t outer,
              uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_outer, bool atom32 = false,
              bool swizzle64 = false);

// Map for the epilogue's TMA stores of 32 x 32 chunks into a row-major [rows, cols] matrix, or false
// if TMA cannot address it (base or row pitch not 16-byte aligned).
bool encode_store_map(CUtensorMap* map, int dtype, void* base, uint64_t rows, uint64_t cols, long long ld);

template <class Cfg>
int launch_cfg(const TcProblem& p, cudaStream_t stream) {
  CUtensorMap ta, tb;
  const uint64_t elt = Cfg::ELT;
  int rc;
  // K-major: inner = K, outer = M (or N); box = one 128-byte row of K x the rows one CTA loads.
  // MN-major: inner = M (or N), outer = K; box = 128 bytes of M/N x BKE rows of K.
  if (Cfg::A_MN)
    rc = encode_2d(&ta, p.op_dtype, p.a, p.g.M, p.g.K, p.a_pitch * elt, Cfg::MN_ATOM, Cfg::BKE, Cfg::MN_BASE32);
  else
    rc = encode_2d(&ta, p.op_dtype, p.a, p.g.K, p.g.M, p.a_pitch * elt, Cfg::BKE, Cfg::BM);
  if (rc != OK) return rc;
  if (Cfg::B_MN)
    rc = encode_2d(&tb, p.op_dtype, p.b, p.g.gate_cols ? 2ull * p.g.gate_cols : p.g.N, p.g.K, p.b_pitch * elt,
                   Cfg::MN_ATOM, Cfg::BKE, Cfg::MN_BASE32);
  else
    rc = encode_2d(&tb, p.op_dtype, p.b, p.g.K, p.g.N, p.b_pitch * elt, Cfg::BKE, Cfg::B_BOX_ROWS);
  if (rc != OK) return rc;

  GemmArgs g = p.g;
  // Outputs of the direct epilogue go through shared memory and TMA stores where TMA can address
  // them; otherwise (and for stream-K partial sums) the epilogue stores from registers.
  CUtensorMap tout = ta, taux = ta;
  g.tma_store = 0;
  if (!g.stream_k && p.allow_tma_store) {
    if (g.out != nullptr && encode_store_map(&tout, g.out_dtype, g.out, g.M, g.N, g.ld_out)) g.tma_store |= 1;
    if (g.aux != nullptr &&
        encode_store_map(&taux, g.out_dtype, g.aux, g.M, g.gate_cols ? 2ull * g.gate_cols : g.N, g.ld_aux))
      g.tma_store |= 2;
  }
  g.tiles_m = (g.M + Cfg::TILE_M - 1) / Cfg::TILE_M;
  g.tiles_n = g.gate_cols ? (g.gate_cols + Cfg::BN / 2 - 1) / (Cfg::BN / 2) : (g.N + Cfg::BN - 1) / Cfg::BN;
  g.k_blocks = (g.K + Cfg::BKE - 1) / Cfg::BKE;
  g.group_m = raster_group_m() / Cfg::CTAS > 0 ? raster_group_m() / Cfg::CTAS : 1;
  const uint32_t fmt = p.op_dtype == DT_F32 ? 2u : (p.op_dtype == DT_BF16 ? 1u : 0u);
  g.idesc = ptx::make_idesc(fmt, Cfg::A_MN ? 1u : 0u, Cfg::B_MN ? 1u : 0u, Cfg::TILE_M, Cfg::BN);

  // Per device: opt in to the large dynamic shared memory and, for CTA pairs, find out how many
  // pairs the device can hold at once.
  static thread_local bool attr_set[64] = {};
  static thread_local int max_workers[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return ERR_LAUNCH;
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(gemm_tcgen05_kernel<Cfg>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Cfg::SMEM_BYTES) != cudaSuccess)
      return ERR_LAUNCH;
    max_workers[dev] = sm_count() / Cfg::CTAS;
    if (Cfg::CTAS > 1) {
      cudaLaunchConfig_t probe = {};
      probe.gridDim = dim3(sm_count() / Cfg::CTAS * Cfg::CTAS);
      probe.blockDim = dim3(Cfg::kThreads);
      probe.dynamicSmemBytes = Cfg::SMEM_BYTES;
      cudaLaunchAttribute attr;
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = Cfg::CTAS;
      attr.val.clusterDim.y = 1;
      attr.val.clusterDim.z = 1;
      probe.attrs = &attr;
      probe.numAttrs = 1;
      int clusters = 0;
      if (cudaOccupancyMaxActiveClusters(&clusters, gemm_tcgen05_kernel<Cfg>, &probe) == cudaSuccess && clusters > 0)
        max_workers[dev] = clusters < max_workers[dev] ? clusters : max_workers[dev];
    }
    attr_set[dev] = true;
  }
  const long long tiles = static_cast<long long>(g.tiles_m) * g.tiles_n;
  const long long work = g.stream_k ? tiles * g.k_blocks : tiles;
  int cap = max_workers[dev];
  int limit = gemm_cta_limit();
  if (p.reserve_sms > 0) {
    const int rest = sm_count() - p.reserve_sms > Cfg::CTAS ? sm_count() - p.reserve_sms : Cfg::CTAS;
    limit = (limit > 0 && limit < rest) ? limit : rest;
  }
  if (limit > 0 && limit / Cfg::CTAS < cap) cap = limit / Cfg::CTAS > 0 ? limit / Cfg::CTAS : 1;
  int workers = static_cast<int>(work < cap ? work : cap);
  if (workers <= 0) return OK;

  // Hybrid schedule: when the last round of whole tiles would be mostly idle (at most 80 % of the
  // workers busy), its tiles' reductions are shared out over all workers instead.
  int tail_tiles = 0;
  CUtensorMap tpartial = ta;
  if (g.gate_cols) {
    // Gated epilogue: whole tiles only, B MN-major; the first half of the saved pre-activation gets a map
    // of its own (see the kernel).
    if (!Cfg::B_MN || g.stream_k) return ERR_BAD_STRIDE;
    if ((g.tma_store & 2) && !encode_store_map(&tpartial, g.out_dtype, g.aux, g.M, g.gate_cols, g.ld_aux))
      g.tma_store &= ~2;
  }
  // Half-width last round: where the last round of whole tiles would fill at most half of the workers,
  // its tiles run as twice as many units of BN / 2 columns, handed out like tiles: that round then
  // takes about half as long (weight-gradient product of 8192 tokens, 4096 -> 4096: 256 pair tiles on
  // 74 CTA pairs = 3 rounds + 34 tiles, 3.5 rounds instead of 4), bit-identical to whole tiles and with
  // the fused epilogue.  Measured on that shape in bursts of 20 launches it is as fast as whole tiles
  // (207 us both; the shared-out round of mode 2: 210 us): the GEMMs run at the power limit, where a
  // half-empty round lets the busy SMs clock higher, so the gain shows only where the last round is
  // emptier.  Forcing it on a full last round (AB200_TAIL_MODE=3) to halve the one epilogue nothing
  // overlaps made the forward pass with bias, gelu and a saved tensor slower (230 vs 217 us): the
  // half-width units fetch the tile's A rows twice.
  // AB200_TAIL_MODE: unset / 0 this rule; 1 whole tiles only; 2 prefer the shared-out round below;
  // 3 half-width units for every last round, full ones too.
  const long long rounds = (tiles + cap - 1) / cap;
  const int last_round = static_cast<int>(tiles - (rounds - 1) * cap);   // tiles in the last round
  const int tail_mode = tail_mode_override();
  if (!g.stream_k && !g.gate_cols && p.allow_split_tail && Cfg::kHalfUnits && tail_mode != 1 && tail_mode != 2 && cap > 1 &&
      (last_round * 2 <= cap || tail_mode == 3)) {
    g.stream_k = 3;
    g.dp_tiles = static_cast<int>(tiles) - last_round;
    // A single round of few tiles: its half-width units can use up to twice as many workers.
    if (rounds == 1) workers = 2 * last_round < cap ? 2 * last_round : cap;
  }
  // Shared-out last round (AB200_TAIL_MODE=2, or where half-width units are not possible).
  if (!g.stream_k && !g.gate_cols && tail_mode != 1 && p.tail_workspace != nullptr && tiles > workers && g.k_blocks >= 16 &&
      workers <= kMaxTailPieces) {
    const int rem = static_cast<int>(tiles % workers);
    // Two slots per worker (its share of the tail touches at most two tiles).
    const long long need = 2ll * workers * Cfg::TILE_M * Cfg::BN * 4;
    if (rem > 0 && rem * 10 <= workers * 8 && need <= p.tail_workspace_bytes &&
        (reinterpret_cast<uintptr_t>(p.tail_workspace) & 15) == 0 &&
        encode_2d(&tpartial, DT_F32, p.tail_workspace, Cfg::BN, 2ull * workers * Cfg::TILE_M, Cfg::BN * 4ull, 32, 32) == OK) {
      tail_tiles = rem;
      g.stream_k = 2;
      g.dp_tiles = static_cast<int>(tiles) - rem;
      g.partial = static_cast<float*>(p.tail_workspace);
    }
  }

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(workers * Cfg::CTAS);
  cfg.blockDim = dim3(Cfg::kThreads);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  if (Cfg::CTAS > 1) {
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = Cfg::CTAS;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
  }
  const cudaError_t err = cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<Cfg>, ta, tb, tout, taux, tpartial, g);
  if (err != cudaSuccess) return ERR_LAUNCH;
  set_last_schedule(g.stream_k);
  if (tail_tiles > 0)
    return launch_hybrid_finish(g, g.dp_tiles, tail_tiles, workers, Cfg::TILE_M, Cfg::BN, stream);
  return OK;
}

// All tile widths of one (element size, majorness) family.  A 32-wide tile is narrower than one
// 128-byte row of an MN-major 16-bit B operand, so it exists only where B is K-major or 4-byte.
// CTA pairs exist for the 256-wide tile-parallel case.
template <int ELT, bool A_MN, bool B_MN>
int launch_family(const TcProblem& p, int bn, cudaStream_t stream) {
  switch (bn) {
    case 32:
      if constexpr (!(B_MN && ELT == 2)) return launch_cfg<GemmCfg<32, ELT, A_MN, B_MN>>(p, stream);
      [[fallthrough]];
    case 64: return launch_cfg<GemmCfg<64, ELT, A_MN, B_MN>>(p, stream);
    case 128: return launch_cfg<GemmCfg<128, ELT, A_MN, B_MN>>(p, stream);
    default:
      if constexpr (!(A_MN && !B_MN)) {
        if (p.allow_pair && !p.g.stream_k && p.g.M > 128)
          return launch_cfg<GemmCfg<256, ELT, A_MN, B_MN, 2>>(p, stream);
      }
      return launch_cfg<GemmCfg<256, ELT, A_MN, B_MN>>(p, stream);
  }
}

}  // namespace ab200
