// Host launcher and C ABI of libneogemm.so (declarations and contracts: include/neogemm.h).
//
// Replaces the reference's host function neoGemmV1 (nemgemmV03.cu:343-391) and its tensor-map
// helpers (nemgemmV03.cu:32-68).  Differences that matter to a caller:
//   * tensor maps are built on the host and passed to the kernel as __grid_constant__ parameters;
//     nothing is cudaMalloc'ed or copied per call (the reference copies each map into device
//     memory, nemgemmV03.cu:60-68) and the cache is keyed by pointer and geometry, not by shape
//     alone (nemgemmV03.cu:359);
//   * arguments are validated and failures come back as status codes (the reference's asserts
//     are compiled out, setup.py:15);
//   * the launch goes to the caller's stream.
// No torch headers here: this file is compiled by nvcc alone and linked with the static CUDA
// runtime; the driver's cuTensorMapEncodeTiled is looked up at run time so the library loads on
// machines without a GPU driver (where every compute entry point reports an error).
#include "../../include/neogemm.h"

#include <cuda_runtime.h>
#include <cudaTypedefs.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <vector>

#include "gemm_sm100.cuh"

namespace neogemm {
namespace {

constexpr int kMaxDevices = 64;
// Bytes reserved at the start of every stream-K workspace for arrival counters (16384 tiles).
constexpr size_t kCounterRegionBytes = 256 * 1024;
// Defaults of the neogemm_set_tuning keys: L2 hint mask, epilogue wait hint (ns), ring wait hint (ns).
constexpr int kDefaultTuning[3] = {0, 2000, 0};
// Two-half tiles: k-blocks issued for half 0 alone when a tile starts.  Half 1 comes back from the
// epilogue ~500 cycles after half 0, so one k-block (512 cycles of tensor work) covers it, and the
// first ring slot is released - and refilled - two k-blocks earlier than with three (8192^3: 924 k
// cycles in the MMA loop against 926 k with two and 928 k with three).
constexpr int kDefaultWidePrologue = 1;
// Throughput assumed for the 256 x 512 pair tile when ranking kernels (TFLOP/s at 8192^3).
constexpr double kWideTileSpeed = 1650.0;
// Microseconds the two-half tile spends handing its accumulators over between tiles, and the
// time the store epilogue of one tile takes (both measured with the phase timers).
constexpr double kHandOverUs = 3.5;
constexpr double kEpilogueUs = 3.0;
// Wave pacing: launches of at least this many waves of whole tiles keep their workers in step
// (see pace_wave in the kernel); each launch takes the next of kPaceSlots counters so that
// launches in flight on different streams do not share one; a worker waits at most this long.
// More than kPaceSlots paced launches in flight at once wrap around and share counters: results
// are unaffected (the wait is soft, nothing depends on it) but a worker that reads a foreign count
// may idle up to the time-out at a wave's start.
// Whole tiles of odd waves walk K backwards (plain round-robin schedules of the TMA-store kernels
// with more than one wave): together with raster groups of 16 tile rows it took 8192^3 from
// 689.3 to 684.2 us in 20-launch bursts and from 761.6 to 757.8 us under seconds of load (cuBLAS
// 690.2 / 763.3 on the same GPU), by way of fewer DRAM reads under the power cap.
constexpr bool kDefaultKAlternate = true;
constexpr int kPaceMinWaves = 8;
constexpr int kPaceSlots = 32;
constexpr int kPaceTimeoutNs = 20000;
// Microseconds a two-pass split-K launch pays on top of its longest k-chunk: publishing the
// partials and the reduction kernel behind the GEMM (used when ranking plans; measured:
// 1024 x 1024 x 8192 in 4 chunks of 32 k-blocks takes 22.6 us where the chunk alone is 13 us).
constexpr double kTwoPassUs = 9.0;
// Widest tile (columns) that has a half-size-ring kernel for two CTAs per SM (five ring stages
// up to 32 columns, four of 24 KB at 64, three of 32 KB at 128) or a tall-tile kernel.
constexpr int kResidentMaxColumns = 128;

// k-blocks per dynamically claimed piece of the stream-K tail pool.
constexpr int kDynPieceKBlocks = 16;
// Row chunks the host entry point cuts the uploaded operand into (one product launch each).
constexpr int kMaxHostChunks = 16;
// Pieces per tile left to the pool unless tuning key 4 says otherwise.
constexpr int kDefaultDynPieces = 1;

// ------------------------------------------------------------------------------------------
// Kernel table
// ------------------------------------------------------------------------------------------
struct KernelEntry {
  int cta_group, block_n, stages, epi, halves;
  int mhalves;  // 128-row blocks of X per CTA tile (2: tall tile sharing Y)
  int per_sm;   // CTAs of this kernel that fit on one SM together (1 or 2)
  const void* fn;
  int smem_bytes;
  int tmem_cols;
  int threads;
};

template <class Cfg>
KernelEntry make_entry() {
  return KernelEntry{Cfg::kCtaGroup, Cfg::BLOCK_N, Cfg::kStages, Cfg::kEpiMode, Cfg::kNHalves,
                     Cfg::kMHalves, Cfg::kCtasPerSm, reinterpret_cast<const void*>(&gemm_bf16_nt_kernel<Cfg>), Cfg::SMEM_TOTAL,
                     Cfg::kTmemCols, Cfg::kThreads};
}

// Stage counts fill the 227 KB of shared memory; a CTA that owns more than half of it is alone on
// its SM, which is what makes its tensor-memory allocation safe from starvation.  The last three
// entries are built to share an SM two at a time and hold at most 128 columns each.
const KernelEntry* kernel_table(int* count) {
  static const KernelEntry table[] = {
      make_entry<GemmConfig<1, 256, 4, kEpiTmaStore>>(),
      make_entry<GemmConfig<1, 128, 6, kEpiTmaStore>>(),
      make_entry<GemmConfig<1, 64, 8, kEpiTmaStore>>(),    // small problems: twice the CTAs
      make_entry<GemmConfig<2, 256, 4, kEpiTmaStore, 2>>(),   // 256 x 512 tile, both accumulators
      make_entry<GemmConfig<2, 256, 6, kEpiTmaStore>>(),
      make_entry<GemmConfig<2, 128, 8, kEpiTmaStore>>(),
      make_entry<GemmConfig<1, 128, 6, kEpiDirect>>(),
      make_entry<GemmConfig<1, 64, 8, kEpiDirect>>(),
      make_entry<GemmConfig<1, 32, 10, kEpiDirect>>(),
      make_entry<GemmConfig<1, 16, 12, kEpiDirect>>(),
      // Half-size rings: two CTAs per SM, one whole tile each (skinny shapes with between one and
      // two tiles per SM, which then need no cut tiles and no closing reduction).
      make_entry<GemmConfig<1, 128, 3, kEpiDirect>>(),
      make_entry<GemmConfig<1, 64, 4, kEpiDirect>>(),
      make_entry<GemmConfig<1, 32, 5, kEpiDirect>>(),
      make_entry<GemmConfig<1, 16, 5, kEpiDirect>>(),
      // Tall tiles: up to 208 rows of X per CTA (a 128-row block and a partly filled one sharing
      // Y), one CTA per SM, ring filled to 227 KB.  Same use as the four above - one resident
      // wave of whole tiles - with the rows spread evenly over the SMs, Y entering an SM once per
      // tile and more bytes of the streamed operand in flight.
      make_entry<GemmConfig<1, 128, 5, kEpiDirect, 1, 2>>(),
      make_entry<GemmConfig<1, 64, 6, kEpiDirect, 1, 2>>(),
      make_entry<GemmConfig<1, 32, 7, kEpiDirect, 1, 2>>(),
      make_entry<GemmConfig<1, 16, 7, kEpiDirect, 1, 2>>(),
      // Tall tiles on CTA pairs: the small operand is split between the two CTAs' rings.
      make_entry<GemmConfig<2, 128, 6, kEpiDirect, 1, 2>>(),
      make_entry<GemmConfig<2, 64, 7, kEpiDirect, 1, 2>>(),
  };
  *count = static_cast<int>(sizeof(table) / sizeof(table[0]));
  return table;
}

const KernelEntry* find_kernel(int cta_group, int block_n, int epi, int halves, int per_sm,
                               int mhalves, int* index) {
  int n;
  const KernelEntry* t = kernel_table(&n);
  for (int i = 0; i < n; ++i) {
    if (t[i].cta_group == cta_group && t[i].block_n == block_n && t[i].epi == epi &&
        t[i].halves == halves && t[i].per_sm == per_sm && t[i].mhalves == mhalves) {
      if (index) *index = i;
      return &t[i];
    }
  }
  return nullptr;
}

// ------------------------------------------------------------------------------------------
// Per-device state
// ------------------------------------------------------------------------------------------
struct DeviceState {
  bool ready = false;
  int init_error = NEOGEMM_OK;
  int sm_count = 0;
  int* status_host = nullptr;  // mapped pinned memory: the kernel writes, the host reads
  int* pace_counters = nullptr;   // kPaceSlots arrival counters, one 128-byte line each, zeroed
  unsigned pace_next = 0;
  int* status_dev = nullptr;
  void* workspace = nullptr;   // library-owned stream-K scratch (grow-only)
  size_t workspace_bytes = 0;
  std::vector<void*> retired_workspaces;   // outgrown scratch buffers, kept for work in flight
  std::mutex host_entry_mu;    // one neogemm_bf16_nt_host call at a time per device
  void* stage[3] = {nullptr, nullptr, nullptr};  // device copies of A, B, C for the host entry
  size_t stage_bytes[3] = {0, 0, 0};
  bool attr_done[32] = {};
  // Host entry point: copy queues for the two PCIe directions and the events that order them.
  cudaStream_t copy_in = nullptr, copy_out = nullptr;
  cudaEvent_t copy_events[2 * kMaxHostChunks + 1] = {};
};

DeviceState g_dev[kMaxDevices];
std::mutex g_mu;
PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;
bool g_encode_looked_up = false;

struct Override {
  int cta_group = -1, block_n = -1, swap = -1, stream_k = -1, group_m = -1, max_ctas = -1;
  int tuning[13] = {-1, -1, -1, -1, -1, -1, -1, -1, -1, -1, -1, -1, -1};   // see neogemm_set_tuning
};
thread_local Override t_override;
thread_local int t_last_config[8] = {0, 0, 0, 0, 0, 0, 0, 0};
thread_local int t_last_store_path = 0;   // see neogemm_last_store_path
thread_local long long* t_timers = nullptr;   // device buffer for phase timers, or null
thread_local size_t t_timers_bytes = 0;

// Must be called with g_mu held.  Returns the state of the current device or nullptr + code.
DeviceState* device_state(int* code) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    cudaGetLastError();
    *code = NEOGEMM_ERR_UNSUPPORTED;
    return nullptr;
  }
  DeviceState& st = g_dev[dev];
  if (st.ready) {
    *code = st.init_error;
    return st.init_error == NEOGEMM_OK ? &st : nullptr;
  }
  st.ready = true;
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
      major != 10 ||
      cudaDeviceGetAttribute(&st.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
    cudaGetLastError();
    st.init_error = NEOGEMM_ERR_UNSUPPORTED;
    *code = st.init_error;
    return nullptr;
  }
  if (!g_encode_looked_up) {
    g_encode_looked_up = true;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) ==
            cudaSuccess && q == cudaDriverEntryPointSuccess) {
      g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
    } else {
      cudaGetLastError();
    }
  }
  if (g_encode == nullptr) {
    st.init_error = NEOGEMM_ERR_DESCRIPTOR;
    *code = st.init_error;
    return nullptr;
  }
  if (cudaHostAlloc(reinterpret_cast<void**>(&st.status_host), 64, cudaHostAllocMapped) !=
          cudaSuccess ||
      cudaHostGetDevicePointer(reinterpret_cast<void**>(&st.status_dev), st.status_host, 0) !=
          cudaSuccess) {
    cudaGetLastError();
    st.init_error = NEOGEMM_ERR_CUDA;
    *code = st.init_error;
    return nullptr;
  }
  std::memset(st.status_host, 0, 64);
  // Arrival counters of the wave pacing; without them the kernels simply do not pace.
  if (cudaMalloc(reinterpret_cast<void**>(&st.pace_counters), kPaceSlots * 128) != cudaSuccess ||
      cudaMemset(st.pace_counters, 0, kPaceSlots * 128) != cudaSuccess) {
    cudaGetLastError();
    st.pace_counters = nullptr;
  }
  *code = NEOGEMM_OK;
  return &st;
}

// ------------------------------------------------------------------------------------------
// Tensor maps
// ------------------------------------------------------------------------------------------
struct MapKey {
  const void* base;
  uint64_t inner, rows, pitch_bytes;
  uint32_t box_rows;
  int for_store;
  bool operator==(const MapKey& o) const {
    return base == o.base && inner == o.inner && rows == o.rows && pitch_bytes == o.pitch_bytes &&
           box_rows == o.box_rows && for_store == o.for_store;
  }
};
struct MapSlot {
  MapKey key;
  CUtensorMap map;
};
thread_local std::vector<MapSlot> t_map_cache;  // most recently used at the back
constexpr size_t kMapCacheSize = 128;

// Row-major bf16 matrix [rows, inner] with row pitch `pitch_bytes`; box = 64 elements (one
// 128-byte swizzle row) x box_rows; out-of-range elements read as zero and are not written.
// Same geometry family as the reference's create_tensor_map (nemgemmV03.cu:32-58), with the
// box height following the tile instead of the fixed 64.
int get_tensor_map(const void* base, uint64_t inner, uint64_t rows, uint64_t pitch_bytes,
                   uint32_t box_rows, int for_store, CUtensorMap* out) {
  // for_store: 1 = store map (no promotion), 2 = store map of an fp32 matrix (`inner` fp32
  // elements per row, box 32 x box_rows: again one 128-byte swizzle row), 1000 + n = store map
  // with a box of n bf16 (a multiple of 8, at most 256) x box_rows, dense in shared memory (no
  // swizzle): the transposed result of a tall tile; loads: 0 = 256-byte L2
  // promotion (default), -1 none, -2 64 B, -3 128 B (tuning key 5).
  const MapKey key{base, inner, rows, pitch_bytes, box_rows, for_store};
  for (size_t i = t_map_cache.size(); i-- > 0;) {
    if (t_map_cache[i].key == key) {
      *out = t_map_cache[i].map;
      return NEOGEMM_OK;
    }
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (pitch_bytes & 15) != 0 ||
      pitch_bytes >= (1ull << 40) || inner == 0 || rows == 0 || inner > 0xffffffffull ||
      rows > 0xffffffffull || box_rows == 0 || box_rows > 256) {
    return NEOGEMM_ERR_UNSUPPORTED;
  }
  cuuint64_t dims[2] = {inner, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {for_store >= 1000 ? static_cast<cuuint32_t>(for_store - 1000)
                                         : for_store == 2 ? 32u : 64u, box_rows};
  if (for_store >= 1000 && (for_store > 1256 || (for_store & 7) != 0)) return NEOGEMM_ERR_UNSUPPORTED;
  cuuint32_t elem_strides[2] = {1, 1};
  CUtensorMap m;
  const CUresult r = g_encode(
      &m, for_store == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
      const_cast<void*>(base), dims, strides, box,
      elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
      for_store >= 1000 ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B,
      for_store >= 1 ? CU_TENSOR_MAP_L2_PROMOTION_NONE
      : for_store == -1 ? CU_TENSOR_MAP_L2_PROMOTION_NONE
      : for_store == -2 ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B
      : for_store == -3 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B
                        : CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return NEOGEMM_ERR_DESCRIPTOR;
  if (t_map_cache.size() >= kMapCacheSize) t_map_cache.erase(t_map_cache.begin());
  t_map_cache.push_back(MapSlot{key, m});
  *out = m;
  return NEOGEMM_OK;
}

// ------------------------------------------------------------------------------------------
// Planning
// ------------------------------------------------------------------------------------------
struct Plan {
  bool swap = false;        // X = the operand that indexes output COLUMNS of the stored matrix
  int cta_group = 1, block_n = 256, epi = kEpiTmaStore;
  int halves = 1;           // 2: 256 x 512 pair tile (two UMMA-N halves sharing X)
  int per_sm = 1;           // 2: half-size rings, two CTAs per SM, one whole tile each
  int mhalves = 1;          // 2: tall tiles sharing Y, one whole tile per CTA
  int tile_rows = 0;        // tall tiles: rows of X per tile (multiple of 8, 136..208)
  bool stream_k = false;
  int sk_first_tile = 0;    // tiles below are handed out round-robin, tiles from here on are cut
  int sk_splits = 0;        // > 0: uniform k-chunks per cut tile (large kernels)
  bool two_pass = false;    // every tile is cut uniformly and a reduction kernel finishes them
  int dyn_ppt = 0, dyn_piece_kb = 0, dyn_static_kb = 0, dyn_pieces = 0;   // dynamic tail pool
  int group_m = 8;
  int num_ctas = 0;
  int Md = 0, Nd = 0;
  int num_m_tiles = 0, num_n_tiles = 0, num_tiles = 0, num_k_blocks = 0;
  int max_contrib = 0;
  size_t counters_bytes = 0, partials_bytes = 0;
  const KernelEntry* kernel = nullptr;
  int kernel_index = -1;
};

int round_block_n(int64_t n) {
  if (n <= 16) return 16;
  if (n <= 32) return 32;
  if (n <= 64) return 64;
  if (n <= 128) return 128;
  return 256;
}

// Into how many equal k-chunks the tiles of a last wave of `rest` tiles (of `workers`) are cut so
// that every worker takes at most one chunk; 0 = leave the wave whole (it is more than half full,
// or K is too short: a chunk must keep at least `min_chunk` k-blocks - 8 for the skinny kernels,
// 16 for the large tiles, whose closing reduction of a cut tile is worth about that much work).
int hybrid_splits(int rest, int workers, int num_k_blocks, int min_chunk = 8) {
  if (rest <= 0) return 0;
  int splits = workers / rest;            // k-chunks per tile so that every worker gets <= 1
  splits = std::min(splits, num_k_blocks / min_chunk);
  return splits >= 2 ? std::min(splits, 8) : 0;
}

// pm x pn is the matrix as stored (row-major, pitch ldc): [M,N] for row-major C, [N,M] for the
// reference's column-major C.
int make_plan(int64_t pm, int64_t pn, int64_t K, int64_t ldc, const void* C, int sm_count,
              const Override& ov, Plan* plan, bool allow_hybrid = true, bool allow_dyn_pool = true,
              int c_elem_bytes = 2) {
  Plan p;
  const bool tma_store_ok = ((ldc * c_elem_bytes) % 16 == 0) &&
                            ((reinterpret_cast<uintptr_t>(C) & 15) == 0);

  // Orientation.  The 128-lane axis of the tensor core wants the long dimension.
  bool swap = (pm <= 128 && pn > pm);
  if (ov.swap >= 0) swap = (ov.swap != 0);
  p.swap = swap;
  const int64_t md = swap ? pn : pm;
  const int64_t nd = swap ? pm : pn;
  if (md > 0x7fffffffll || nd > 0x7fffffffll) return NEOGEMM_ERR_UNSUPPORTED;
  p.Md = static_cast<int>(md);
  p.Nd = static_cast<int>(nd);

  int block_n = round_block_n(nd);
  if (ov.block_n > 0) block_n = ov.block_n;
  int cta_group = 1;
  if (ov.cta_group > 0) cta_group = ov.cta_group;
  int epi = kEpiDirect;
  if (!swap && tma_store_ok && block_n >= 128) epi = kEpiTmaStore;
  // A handful of output tiles under a long K (512 x 512 x 8192: 16 tiles of 128 x 128 on 148
  // SMs): 64-column direct-store tiles, which the schedule below cuts into k-chunks, one per CTA.
  // Their partials are small (32 KB) and every cut tile has its own finisher, so the closing sums
  // stay short.  Measured: 512 x 512 x 8192 37.8 -> 18.7 us, 256 x 256 x 4096 21.4 -> 15.6 us;
  // with more tiles than an eighth of the SMs the whole tiles win (1536 x 1024 x 3072).
  // (Only with the two-pass split-K switched off, tuning key 11 = 0: cutting the wide tiles and
  // summing them in a second kernel is faster still - 512 x 512 x 8192 then runs as 4 pair tiles
  // in 8 chunks.)
  if (epi == kEpiTmaStore && ov.block_n <= 0 && ov.cta_group <= 0 && ov.stream_k != 0 &&
      ov.tuning[11] == 0 &&
      ov.tuning[3] != 1 && allow_hybrid && (K + 63) / 64 >= 64 &&
      ((md + 127) / 128) * ((nd + 127) / 128) * 8 <= sm_count) {
    epi = kEpiDirect;
    block_n = 64;
  }
  // The direct-store epilogue exists for 16..128 columns only: outputs whose pitch or address
  // rules out the TMA store (N % 8 != 0 for a packed row-major C) take the 128-wide tile.
  if (epi == kEpiDirect && block_n > 128) block_n = 128;
  if (cta_group == 2 && (epi != kEpiTmaStore || block_n < 128)) cta_group = 1;
  if (epi == kEpiTmaStore) {
    // Choose among the TMA-store kernels by estimated time: waves of tiles over the
    // workers (SMs, or SM pairs) times the work of one tile per SM, divided by the throughput
    // each kernel reached at 8192^3 on a B200 (TFLOP/s, measured).  Overrides pin a field.
    struct Candidate { int cta_group, block_n, halves; double speed; };
    const Candidate candidates[5] = {{2, 256, 2, kWideTileSpeed}, {2, 256, 1, 1570.0},
                                     {1, 256, 1, 1430.0}, {1, 128, 1, 1170.0}, {2, 128, 1, 975.0}};
    double best = 0.0;
    int best_group = cta_group, best_n = block_n, best_halves = 1;
    const int wide = ov.tuning[3];   // -1 auto, 0 never, 1 always (when the shape allows)
    for (const Candidate& c : candidates) {
      // An explicit tile-width override means the one-half kernels unless the wide tile is forced.
      if (c.halves == 2 && (wide == 0 || ov.cta_group == 1 || (ov.block_n > 0 && wide != 1) ||
                            (ov.block_n > 0 && ov.block_n != 256)))
        continue;
      if (c.halves == 1 && wide == 1 && nd > 256 && ov.cta_group != 1 &&
          (ov.block_n < 0 || ov.block_n == 256))
        continue;
      if (ov.cta_group > 0 && c.cta_group != ov.cta_group) continue;
      if (ov.block_n > 0 && c.block_n != ov.block_n) continue;
      if (c.block_n > block_n && ov.block_n < 0) continue;   // nd <= 128: no 256-wide tile
      if (c.halves == 2 && nd <= 256) continue;
      const int64_t workers = std::max(1, sm_count / c.cta_group);
      const int64_t tm = 128 * c.cta_group;
      const int64_t tile_n = static_cast<int64_t>(c.block_n) * c.halves;
      const int64_t tiles = ((md + tm - 1) / tm) * ((nd + tile_n - 1) / tile_n);
      const int rest = static_cast<int>(tiles % workers);
      double waves = static_cast<double>(tiles / workers);
      double extra_us = 0.0;
      if (rest > 0) {
        const bool may_cut = allow_hybrid && ov.stream_k != 0 && c.halves == 1;
        int cut = 0;
        if (may_cut && tiles >= workers) {
          cut = hybrid_splits(rest, static_cast<int>(workers), static_cast<int>((K + 63) / 64), 16);
        } else if (may_cut && ov.tuning[11] != 0) {
          // fewer tiles than workers: every tile in `cut` chunks, summed by a second kernel -
          // where that beats the whole tiles (the schedule below applies the same test)
          cut = hybrid_splits(rest, static_cast<int>(workers), static_cast<int>((K + 63) / 64), 8);
          if (cut > 0) {
            const double t_whole = 2.0 * 128.0 * c.cta_group * static_cast<double>(c.block_n) *
                                   static_cast<double>(K) /
                                   (c.speed * 1e6 / std::max(1, sm_count / c.cta_group));
            if (ov.stream_k < 0 &&
                t_whole / cut * 1.05 + kTwoPassUs >= std::max(t_whole, kEpilogueUs))
              cut = 0;
            else
              extra_us = kTwoPassUs;
          }
        }
        waves += cut > 0 ? 1.0 / cut + 0.05 : 1.0;
      }
      // Time of one tile on one worker at that kernel's throughput, in microseconds, plus what
      // the epilogue adds: the two-half tile exposes the hand-over between tiles (no second
      // accumulator), the others hide the epilogue unless the main loop is shorter than it.
      const double workers_full = std::max(1, sm_count / c.cta_group);
      const double t_main = 2.0 * static_cast<double>(tm) * static_cast<double>(tile_n) *
                            static_cast<double>(K) / (c.speed * 1e6 / workers_full);
      const double t_tile = (c.halves == 2) ? t_main + kHandOverUs : std::max(t_main, kEpilogueUs);
      // (the last term only breaks ties between kernels whose main loops all hide behind one
      // epilogue: tiny problems take the kernel with the least work per CTA)
      const double cost = waves * t_tile + extra_us + 0.01 * t_main;
      if (best == 0.0 || cost < best) {
        best = cost;
        best_group = c.cta_group;
        best_n = c.block_n;
        best_halves = c.halves;
      }
    }
    cta_group = best_group;
    block_n = best_n;
    p.halves = best_halves;
    // Small problems: when the 128 x 128 tiles would leave at least half of the SMs idle, 128 x 64
    // tiles put twice as many to work.  Such launches are bound by the latency of the loads, not
    // by the tensor pipe (about 1.3 us from issue to landing even out of L2): the narrower tile
    // has a deeper ring (8 slots of 24 KB), half the MMA work and half the epilogue per CTA.
    // Tuning key 12: -1 as described, 0 never, 1 whenever the 128 x 128 kernel would be used.
    if (cta_group == 1 && block_n == 128 && p.halves == 1 && ov.block_n <= 0 && ov.tuning[12] != 0) {
      const int64_t tiles128 = ((md + 127) / 128) * ((nd + 127) / 128);
      // (up to K = 2048: few tiles under a longer K are cut into k-chunks instead, below)
      if (ov.tuning[12] == 1 || (2 * tiles128 <= sm_count && (K + 63) / 64 <= 32)) block_n = 64;
    }
  }
  p.block_n = block_n;
  p.cta_group = cta_group;
  p.epi = epi;
  // Skinny shapes with more 128-row tiles than SMs (decode: 224 on 148) run as ONE wave of whole
  // tiles where that is possible: every CTA streams its rows of X over all of K, nothing is cut,
  // nothing has to be summed at the end.  Two kernels can do that.
  //  * Tall tiles (the default): the rows are dealt out evenly, ceil(rows / SMs) rounded up to a
  //    multiple of 8 per CTA - 200 at 28672 rows, on 144 CTAs - as long as that is at most 208
  //    (a 128-row MMA block and a partly used second one; cuBLAS' M=16 kernel is of the same
  //    family: nvjet_tst_256x16, 112 whole tiles of 256 rows).  Every SM then has loads of the
  //    streamed operand in flight (its latency under load is about 3 us, so the bytes in flight
  //    are what sets the rate), the small operand enters an SM once per tile instead of once per
  //    128 rows (at M=128 it is as large as the streamed one), and one CTA per SM has the whole
  //    227 KB for its ring.
  //  * 128-row tiles with two CTAs per SM and half-size rings, when there are at most two such
  //    tiles per SM and the tall tiles would have to be higher than 208 rows.
  // Tuning key 7: -1 as described, 0 neither (stream-K), 1 two CTAs per SM whenever the kernel
  // exists and the tiles fit, 2 tall tiles for any row count up to 208 rows per SM, 3 and 4 as
  // -1 with another store path for tall tiles (see gemm_device).
  int mhalves = 1, tile_rows = 0;
  bool two_per_sm_auto = false;
  {
    const int64_t n_tiles = (nd + block_n - 1) / block_n;
    const int64_t tiles128 = ((md + 127) / 128) * n_tiles;
    const int64_t share = (md * n_tiles + sm_count - 1) / sm_count;      // rows per SM, evenly
    const int64_t rows = std::max<int64_t>(136, (share + 7) / 8 * 8);
    const bool one_wave_ok = epi == kEpiDirect && cta_group == 1 &&
                             block_n <= kResidentMaxColumns && ov.stream_k <= 0 &&
                             ov.max_ctas <= 0 && (K + 63) / 64 >= 16;
    const bool tall_fits = rows <= 208 && ((md + rows - 1) / rows) * n_tiles <= sm_count;
    if (one_wave_ok && tall_fits &&
        (((ov.tuning[7] < 0 || ov.tuning[7] >= 3) && tiles128 > sm_count) || ov.tuning[7] == 2)) {
      mhalves = 2;
      tile_rows = static_cast<int>(rows);
      // From 64 columns on the small operand is worth splitting between two CTAs: pairs of
      // tall tiles (2 x tile_rows rows per pair), provided the pairs still fit in one wave.
      const int64_t pair_tiles = ((md + 2 * rows - 1) / (2 * rows)) * n_tiles;
      if (block_n >= 64 && ov.cta_group != 1 && 2 * pair_tiles <= sm_count) cta_group = 2;
    } else if (one_wave_ok && (ov.tuning[7] < 0 || ov.tuning[7] >= 3) && tiles128 > sm_count &&
               tiles128 <= 2ll * sm_count) {
      two_per_sm_auto = true;
    }
  }
  p.mhalves = mhalves;
  p.tile_rows = tile_rows;
  p.cta_group = cta_group;   // (pairs of tall tiles were decided just above)
  const int tile_m = mhalves == 2 ? tile_rows * cta_group : 128 * cta_group;
  p.num_m_tiles = static_cast<int>((md + tile_m - 1) / tile_m);
  const int tile_n = block_n * p.halves;
  p.num_n_tiles = static_cast<int>((nd + tile_n - 1) / tile_n);
  const int64_t tiles = static_cast<int64_t>(p.num_m_tiles) * p.num_n_tiles;
  if (tiles > 0x3fffffffll) return NEOGEMM_ERR_UNSUPPORTED;

  // The other one-wave plan for skinny shapes (see above): 128-row tiles, two CTAs per SM with
  // half-size rings.  Measured before tall tiles existed (CUDA-graph replays, M x 28672 x 8192,
  // against stream-K on 148 CTAs): M=16 78.3 -> 74.2 us, M=32 81.8 -> 76.9 us, M=64 84.4 -> 83.0 us
  // (K=4096: 48.2 -> 40.2 us), M=128 87.8 -> 82.8 us, M=96 91.6 -> 84.3 us.  Picked only on
  // request (tuning key 7 = 1), whenever the kernel exists and all tiles fit at once.
  int per_sm = 1;
  if (epi == kEpiDirect && cta_group == 1 && mhalves == 1 && ov.stream_k <= 0 &&
      ov.max_ctas <= 0 && tiles <= 2ll * sm_count && (K + 63) / 64 >= 16 &&
      block_n <= kResidentMaxColumns && (ov.tuning[7] == 1 || two_per_sm_auto))
    per_sm = 2;
  p.per_sm = per_sm;
  p.kernel = find_kernel(cta_group, block_n, epi, p.halves, per_sm, mhalves, &p.kernel_index);
  if (p.kernel == nullptr) return NEOGEMM_ERR_UNSUPPORTED;

  p.num_tiles = static_cast<int>(tiles);
  p.num_k_blocks = static_cast<int>((K + 63) / 64);

  // Raster group height (tile rows walked before moving one tile column on).  Pair tiles: 8 rows
  // (2048 rows of X) keep a wave near square; from 8192 rows on the groups are 16 tall: tall
  // problems re-read all of Y once per group (measured at 65536 x 8192 x 8192: +5 %), and with
  // the K direction alternating between waves 16 is the best height at 8192^3 too (12: 685.4 us,
  // 16: 684.2, 20: 686.3, 24: 691.2).
  p.group_m = (cta_group == 2) ? ((p.num_m_tiles >= 32) ? 16 : 8) : 16;
  if (ov.group_m > 0) p.group_m = ov.group_m;
  p.group_m = std::max(1, std::min(p.group_m, p.num_m_tiles));

  const int workers_max = std::max(1, per_sm * sm_count / cta_group);
  int workers = workers_max;
  if (ov.max_ctas > 0) workers = std::max(1, std::min(workers, ov.max_ctas / cta_group));

  // Schedule.
  //  * Direct-store (skinny) kernels: stream-K over ALL tiles when whole tiles cannot fill or
  //    balance the machine and there is enough K to cut.
  //  * TMA-store kernels: whole waves of tiles go round-robin; a last, partly filled wave is cut
  //    stream-K style among all workers when that shortens the launch (wave quantisation:
  //    4096^3 is 3.46 waves of pair tiles).
  bool stream_k = false;
  int sk_first = 0, sk_splits = 0;
  if (per_sm == 2 || mhalves == 2) {
    // one whole tile per CTA, all resident at once
  } else if (epi == kEpiDirect) {
    if (p.num_tiles < workers) {
      // Fewer tiles than SMs: cut every tile into the same few k-chunks, one per CTA.  Few
      // contributors per tile keep the closing reduction short (a contiguous cut of such a
      // small unit space would give each tile five or more).
      sk_splits = ov.stream_k != 0 ? hybrid_splits(p.num_tiles, workers, p.num_k_blocks) : 0;
      stream_k = sk_splits > 0;
      if (ov.stream_k > 0 && !stream_k) stream_k = true;   // forced: contiguous ranges
    } else {
      // More tiles than SMs but not a whole number of waves (the decode shapes: 224 tiles on
      // 148 SMs): equal contiguous ranges, provided every CTA keeps a long enough run.
      const int64_t per_cta = static_cast<int64_t>(p.num_tiles) * p.num_k_blocks / workers;
      stream_k = (block_n <= 128) && (per_cta >= 32) && (p.num_tiles % workers != 0) &&
                 (p.num_tiles < 8 * workers);
      if (ov.stream_k >= 0) stream_k = (ov.stream_k != 0);
    }
  } else {
    // Only behind at least one whole wave: the cut tiles are done first, and their closing
    // reduction then hides under the whole tiles that follow.
    const int rest = p.num_tiles % workers;
    if (p.num_tiles >= workers) {
      sk_splits = allow_hybrid && ov.stream_k != 0 && p.halves == 1
          ? hybrid_splits(rest, workers, p.num_k_blocks, 16) : 0;
      sk_first = p.num_tiles - rest;
    } else if (allow_hybrid && ov.stream_k != 0 && p.halves == 1 && ov.tuning[11] != 0) {
      // Fewer tiles than workers (few wide tiles under a long K): every tile in the same number
      // of k-chunks, one per worker; the reduction kernel behind the launch sums them.  Only
      // where the shorter main loop pays for the second pass (or on request).
      sk_splits = hybrid_splits(p.num_tiles, workers, p.num_k_blocks, 8);
      sk_first = 0;
      const double speed = cta_group == 2 ? (block_n == 256 ? 1570.0 : 975.0)
                                          : (block_n == 256 ? 1430.0 : block_n == 128 ? 1170.0 : 600.0);
      const double t_tile = 2.0 * tile_m * static_cast<double>(block_n) * static_cast<double>(K) /
                            (speed * 1e6 / std::max(1, sm_count / cta_group));
      if (sk_splits > 0 && ov.stream_k < 0 &&
          t_tile / sk_splits * 1.05 + kTwoPassUs >= std::max(t_tile, kEpilogueUs))
        sk_splits = 0;
    }
    stream_k = sk_splits > 0;
  }
  const int sk_tiles = stream_k ? p.num_tiles - sk_first : 0;
  if (stream_k &&
      (static_cast<size_t>(sk_tiles) * cta_group * 4 + 1) * sizeof(int) > kCounterRegionBytes) {
    if (ov.stream_k > 0) return NEOGEMM_ERR_UNSUPPORTED;
    stream_k = false;
  }
  p.stream_k = stream_k;
  p.sk_first_tile = stream_k ? sk_first : 0;
  p.sk_splits = stream_k ? sk_splits : 0;
  // All tiles cut uniformly: nothing follows the cut tiles that could hide a closing sum inside
  // the GEMM kernel, so the sums go to a second kernel that uses every SM (tuning key 11 = 0:
  // the last contributor to arrive sums, as for a cut last wave).
  p.two_pass = stream_k && sk_splits > 0 && sk_first == 0 && ov.tuning[11] != 0;
  if (stream_k) {
    if (sk_splits > 0) {
      p.max_contrib = sk_splits;
      if (sk_first == 0) workers = std::min(workers, sk_tiles * sk_splits);   // one chunk per CTA
    } else {
      // Dynamic tail pool: with enough K, the last 16 or 32 k-blocks of every tile are left out
      // of the static ranges and claimed at run time in pieces of 16 (tuning key 4: 0 = off).
      int static_kb = p.num_k_blocks;
      // Measured on the decode shapes: one piece per tile pays for 16 output columns (2 % faster
      // at M=16); from 32 columns on the extra partial round trips cost more than the balancing
      // gains (M=32: 78.8 us without, 83.2 us with).
      const int want = ov.tuning[4] >= 0 ? ov.tuning[4] : (block_n <= 16 ? kDefaultDynPieces : 0);
      if (want > 0 && p.num_k_blocks >= 64 && cta_group == 1 && allow_dyn_pool) {
        p.dyn_ppt = std::min(want, 4);
        p.dyn_piece_kb = kDynPieceKBlocks;
        p.dyn_static_kb = p.num_k_blocks - p.dyn_ppt * kDynPieceKBlocks;
        p.dyn_pieces = sk_tiles * p.dyn_ppt;
        static_kb = p.dyn_static_kb;
      }
      const int64_t static_units = static_cast<int64_t>(sk_tiles) * static_kb;
      workers = static_cast<int>(std::min<int64_t>(workers, static_units));
      const int64_t per = std::max<int64_t>(1, static_units / workers);
      p.max_contrib = static_cast<int>((static_kb + per - 1) / per) + 1 + p.dyn_ppt;
    }
    // The arrival counters always occupy the same fixed region at the start of a workspace, so
    // that launches of different shapes sharing one workspace never see each other's partials
    // where they expect zeroed counters.
    p.counters_bytes = kCounterRegionBytes;
    p.partials_bytes = static_cast<size_t>(sk_tiles) * p.max_contrib * block_n * tile_m *
                       sizeof(float);
  } else {
    workers = std::min(workers, p.num_tiles);
  }
  p.num_ctas = workers * cta_group;
  *plan = p;
  return NEOGEMM_OK;
}

int validate(const void* A, const void* B, const void* C, int64_t M, int64_t N, int64_t K,
             int64_t lda, int64_t ldb, int64_t ldc, int c_col_major, int c_elem_bytes = 2) {
  if (M < 0 || N < 0 || K < 0) return NEOGEMM_ERR_BAD_ARG;
  if (M == 0 || N == 0) return NEOGEMM_OK;
  if (C == nullptr) return NEOGEMM_ERR_BAD_ARG;
  if (ldc < (c_col_major ? M : N)) return NEOGEMM_ERR_BAD_ARG;
  if (K == 0) return NEOGEMM_OK;
  if (A == nullptr || B == nullptr) return NEOGEMM_ERR_BAD_ARG;
  if (lda < K || ldb < K) return NEOGEMM_ERR_BAD_ARG;
  if (K % 8 != 0 || lda % 8 != 0 || ldb % 8 != 0) return NEOGEMM_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(A) & 15) != 0 || (reinterpret_cast<uintptr_t>(B) & 15) != 0)
    return NEOGEMM_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(C) & static_cast<uintptr_t>(c_elem_bytes - 1)) != 0)
    return NEOGEMM_ERR_UNSUPPORTED;
  if (M > 0x7fffffffll || N > 0x7fffffffll || K > 0x7fffffffll) return NEOGEMM_ERR_UNSUPPORTED;
  return NEOGEMM_OK;
}

// Library-owned stream-K scratch.  It only ever grows, and a buffer it has outgrown stays
// allocated: launches still queued, and CUDA graphs captured earlier with workspace == NULL,
// keep pointing at the old one (sizes at least double, so the retired buffers add up to less than
// the live one).  Growing means cudaMalloc + cudaMemset, which a capturing stream does not allow:
// then the call is refused and the caller makes one plain call first, or passes its own workspace.
int ensure_workspace(DeviceState* st, size_t bytes, cudaStream_t stream) {
  if (bytes <= st->workspace_bytes) return NEOGEMM_OK;
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &capturing) != cudaSuccess) {
    cudaGetLastError();
    return NEOGEMM_ERR_CUDA;
  }
  if (capturing != cudaStreamCaptureStatusNone) return NEOGEMM_ERR_WORKSPACE;
  const size_t want = std::max({bytes, 2 * st->workspace_bytes, static_cast<size_t>(64) << 20});
  void* fresh = nullptr;
  if (cudaMalloc(&fresh, want) != cudaSuccess) {
    cudaGetLastError();
    return NEOGEMM_ERR_WORKSPACE;
  }
  if (cudaMemset(fresh, 0, want) != cudaSuccess) {
    cudaGetLastError();
    cudaFree(fresh);
    return NEOGEMM_ERR_WORKSPACE;
  }
  if (st->workspace != nullptr) st->retired_workspaces.push_back(st->workspace);
  st->workspace = fresh;
  st->workspace_bytes = want;
  return NEOGEMM_OK;
}

int launch(DeviceState* st, const Plan& plan, const CUtensorMap& mx, const CUtensorMap& my,
           const CUtensorMap& md, const GemmParams& params, cudaStream_t stream,
           bool overlap_setup = true) {
  const KernelEntry* k = plan.kernel;
  if (!st->attr_done[plan.kernel_index]) {
    if (cudaFuncSetAttribute(k->fn, cudaFuncAttributeMaxDynamicSharedMemorySize, k->smem_bytes) !=
        cudaSuccess) {
      cudaGetLastError();
      return NEOGEMM_ERR_LAUNCH;
    }
    st->attr_done[plan.kernel_index] = true;
  }
  cudaLaunchConfig_t cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(static_cast<unsigned>(plan.num_ctas), 1, 1);
  cfg.blockDim = dim3(static_cast<unsigned>(k->threads), 1, 1);
  cfg.dynamicSmemBytes = static_cast<size_t>(k->smem_bytes);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int nattr = 0;
  if (k->cta_group == 2) {
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    nattr = 1;
  }
  if (overlap_setup) {
    // Programmatic dependent launch: this kernel's CTAs may be placed and run their set-up
    // (barrier initialisation, tensor-memory allocation, descriptor prefetch) while the previous
    // kernel of the stream drains; the kernel waits for that kernel's completion before its first
    // access to global memory (griddep_wait), so ordering of data is unchanged.
    attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[nattr].val.programmaticStreamSerializationAllowed = 1;
    ++nattr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = nattr;
  void* args[4] = {const_cast<CUtensorMap*>(&mx), const_cast<CUtensorMap*>(&my),
                   const_cast<CUtensorMap*>(&md), const_cast<GemmParams*>(&params)};
  if (cudaLaunchKernelExC(&cfg, k->fn, args) != cudaSuccess) {
    cudaGetLastError();
    return NEOGEMM_ERR_LAUNCH;
  }
  return NEOGEMM_OK;
}

// Second pass of a two-pass split-K launch (see splitk_reduce_kernel): right behind the GEMM
// kernel on the same stream, with the same set-up overlap.
int launch_reduce(const DeviceState* st, const Plan& plan, const GemmParams& params,
                  cudaStream_t stream, bool overlap_setup = true) {
  const int tile_m = 128 * plan.cta_group;
  const long long items = static_cast<long long>(plan.num_tiles) * tile_m * (plan.block_n / 8);
  const long long blocks = std::min<long long>((items + 255) / 256, 8ll * st->sm_count);
  cudaLaunchConfig_t cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(static_cast<unsigned>(std::max<long long>(1, blocks)), 1, 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = overlap_setup ? 1 : 0;
  int tm = tile_m, bn = plan.block_n;
  void* args[3] = {const_cast<GemmParams*>(&params), &tm, &bn};
  if (cudaLaunchKernelExC(&cfg, reinterpret_cast<const void*>(&splitk_reduce_kernel), args) !=
      cudaSuccess) {
    cudaGetLastError();
    return NEOGEMM_ERR_LAUNCH;
  }
  return NEOGEMM_OK;
}

// Optional fused epilogue: C = act(alpha * A B^T + beta * C + bias).
// A tall tile hands a transposed bf16 result (rows of D contiguous in memory: the operands were
// swapped) to the TMA unit instead of storing it from registers; the map's box is the whole tile,
// tile_rows rows of D (contiguous bytes) by the tile's columns.  Tile heights are multiples of 8,
// so every box starts on a 16-byte boundary and its rows are whole 16-byte units.
bool tall_tile_tma_store(const Plan& plan, const void* C, int64_t ldc, int c_elem) {
  return plan.mhalves == 2 && plan.swap && c_elem == 2 && (ldc & 7) == 0 &&
         (reinterpret_cast<uintptr_t>(C) & 15) == 0 && (plan.tile_rows & 7) == 0;
}

struct Fusion {
  bool on = false;
  float alpha = 1.f, beta = 0.f;
  const void* bias = nullptr;   // bf16[N] or null
  int activation = 0;           // 0 none, 1 ReLU, 2 GELU (tanh form)
  bool out_f32 = false;         // C holds fp32: the result is stored unrounded
};

int gemm_device(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                int64_t lda, int64_t ldb, int64_t ldc, int c_col_major, void* workspace,
                size_t workspace_bytes, cudaStream_t stream, const Fusion& fusion = Fusion()) {
  const int c_elem = fusion.out_f32 ? 4 : 2;
  int rc = validate(A, B, C, M, N, K, lda, ldb, ldc, c_col_major, c_elem);
  if (rc != NEOGEMM_OK) return rc;
  if (M == 0 || N == 0) return NEOGEMM_OK;
  if (fusion.on && K == 0) return NEOGEMM_ERR_UNSUPPORTED;

  DeviceState* st;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    st = device_state(&rc);
  }
  if (st == nullptr) return rc;
  if (st->status_host[0] != 0) return NEOGEMM_ERR_DEVICE_TIMEOUT;

  const int64_t pm = c_col_major ? N : M;
  const int64_t pn = c_col_major ? M : N;
  if (K == 0) {
    if (cudaMemset2DAsync(C, static_cast<size_t>(ldc) * 2, 0, static_cast<size_t>(pn) * 2,
                          static_cast<size_t>(pm), stream) != cudaSuccess) {
      cudaGetLastError();
      return NEOGEMM_ERR_CUDA;
    }
    return NEOGEMM_OK;
  }
  const void* U = c_col_major ? B : A;   // rows of the stored matrix
  const void* V = c_col_major ? A : B;   // columns of the stored matrix
  const int64_t ldu = c_col_major ? ldb : lda;
  const int64_t ldv = c_col_major ? lda : ldb;

  Plan plan;
  Override ov = t_override;
  if (fusion.out_f32) ov.tuning[3] = 0;   // two-half tiles keep their result packed as bf16
  rc = make_plan(pm, pn, K, ldc, C, st->sm_count, ov, &plan, true, true, c_elem);
  if (rc != NEOGEMM_OK) return rc;

  const void* X = plan.swap ? V : U;
  const void* Y = plan.swap ? U : V;
  const int64_t ldx = plan.swap ? ldv : ldu;
  const int64_t ldy = plan.swap ? ldu : ldv;

  CUtensorMap mx, my, md;
  std::memset(&md, 0, sizeof(md));
  // tuning key 5: 0 = none, 1 = 64 B, 2 = 128 B, 3 (and default) = 256 B promotion of loads
  const int promo = (t_override.tuning[5] >= 0 && t_override.tuning[5] < 3)
      ? -1 - t_override.tuning[5] : 0;
  rc = get_tensor_map(X, static_cast<uint64_t>(K), static_cast<uint64_t>(plan.Md),
                      static_cast<uint64_t>(ldx) * 2,
                      plan.mhalves == 2 ? static_cast<uint32_t>(plan.tile_rows) : 128u, promo, &mx);
  if (rc != NEOGEMM_OK) return rc;
  rc = get_tensor_map(Y, static_cast<uint64_t>(K), static_cast<uint64_t>(plan.Nd),
                      static_cast<uint64_t>(ldy) * 2,
                      static_cast<uint32_t>(plan.block_n / plan.cta_group), promo, &my);
  if (rc != NEOGEMM_OK) return rc;
  if (plan.epi == kEpiTmaStore) {
    rc = get_tensor_map(C, static_cast<uint64_t>(plan.Nd), static_cast<uint64_t>(plan.Md),
                        static_cast<uint64_t>(ldc) * c_elem, 32, fusion.out_f32 ? 2 : 1, &md);
    if (rc != NEOGEMM_OK) return rc;
  }
  // Tuning key 7 = 3: tall tiles as by default, but stored from registers; 4: stored through the
  // TMA unit, but the pair kernel of 128 columns keeps the operands' usual roles.
  bool tall_tma = tall_tile_tma_store(plan, C, ldc, c_elem) && t_override.tuning[7] != 3;
  bool tall_flip = tall_tma && plan.cta_group == 2 && plan.block_n == 128 && !fusion.on &&
                   t_override.tuning[7] != 4;
  if (tall_tma) {
    rc = get_tensor_map(C, static_cast<uint64_t>(plan.Md), static_cast<uint64_t>(plan.Nd),
                        static_cast<uint64_t>(ldc) * 2,
                        tall_flip ? 32u : static_cast<uint32_t>(plan.block_n),
                        1000 + plan.tile_rows, &md);
    if (rc != NEOGEMM_OK) tall_tma = tall_flip = false;   // stores from registers serve any C
  }

  GemmParams params;
  std::memset(&params, 0, sizeof(params));
  params.Md = plan.Md;
  params.Nd = plan.Nd;
  params.K = static_cast<int>(K);
  params.num_m_tiles = plan.num_m_tiles;
  params.num_n_tiles = plan.num_n_tiles;
  params.num_tiles = plan.num_tiles;
  params.num_k_blocks = plan.num_k_blocks;
  params.group_m = plan.group_m;
  params.tile_rows = plan.tile_rows;
  // Skinny shapes with a single tile column read every row panel of X exactly once: mark those
  // loads evict-first and the small, endlessly re-read Y evict-last, so that the stream does not
  // push Y and the stream-K partials out of L2 (measured: 5 % at M=16, 9 % at M=128 on the decode
  // shapes).
  const int default_hints = (plan.epi == kEpiDirect && plan.num_n_tiles == 1) ? 24 : kDefaultTuning[0];
  params.l2_hints = (t_override.tuning[0] >= 0 ? t_override.tuning[0] : default_hints) |
                    (tall_flip ? 64 : tall_tma ? 32 : 0);
  params.epi_wait_hint_ns = t_override.tuning[1] >= 0 ? t_override.tuning[1] : kDefaultTuning[1];
  params.main_wait_hint_ns = t_override.tuning[2] >= 0 ? t_override.tuning[2] : kDefaultTuning[2];
  params.wide_prologue = t_override.tuning[6] >= 0 ? t_override.tuning[6] : kDefaultWidePrologue;
  params.out = static_cast<__nv_bfloat16*>(C);
  params.out_stride_r = plan.swap ? 1 : ldc;
  params.out_stride_c = plan.swap ? ldc : 1;
  params.stream_k = plan.stream_k ? 1 : 0;
  params.sk_first_tile = plan.sk_first_tile;
  params.sk_splits = plan.sk_splits;
  params.dyn_pieces = plan.dyn_pieces;
  params.dyn_ppt = plan.dyn_ppt;
  params.dyn_piece_kb = plan.dyn_piece_kb;
  params.dyn_static_kb = plan.dyn_static_kb;
  params.max_contrib = plan.max_contrib;
  params.sk_two_pass = plan.two_pass ? 1 : 0;
  params.status = st->status_dev;
  // Tuning key 8: wave pacing -1 auto (many waves of whole tiles), 0 off, 1 whenever applicable.
  {
    const int workers = plan.num_ctas / plan.cta_group;
    const int want = t_override.tuning[8];
    const bool applicable = !plan.stream_k && plan.epi == kEpiTmaStore &&
                            st->pace_counters != nullptr && plan.num_tiles > workers;
    if (applicable && want != 0 && (want == 1 || plan.num_tiles >= kPaceMinWaves * workers)) {
      std::lock_guard<std::mutex> lock(g_mu);
      params.pace_counter = st->pace_counters + (st->pace_next++ % kPaceSlots) * 32;
      params.pace_timeout_ns = kPaceTimeoutNs;
    }
  }
  // Tuning key 9: alternate the K direction from wave to wave (-1 auto: plain round-robin
  // schedules of TMA-store kernels with more than one wave; 0 off; 1 on for every schedule).
  {
    const int want = t_override.tuning[9];
    const int workers = plan.num_ctas / plan.cta_group;
    params.k_alternate = (want == 1 || (want < 0 && kDefaultKAlternate && !plan.stream_k &&
                                        plan.epi == kEpiTmaStore && plan.num_tiles > workers)) ? 1 : 0;
  }
  if (fusion.on) {
    params.fuse = 1;
    params.alpha = fusion.alpha;
    params.beta = fusion.beta;
    params.c_in = static_cast<const __nv_bfloat16*>(C);
    if (fusion.out_f32) {
      params.out32 = static_cast<float*>(C);
      params.c_in32 = static_cast<const float*>(C);
    }
    params.bias = static_cast<const __nv_bfloat16*>(fusion.bias);
    // The bias runs along N.  N is the row axis of D when exactly one of "column-major C" and
    // "operands swapped" holds.
    params.bias_on_rows = ((c_col_major != 0) != plan.swap) ? 1 : 0;
    params.activation = fusion.activation;
  }
  params.timers = nullptr;
  if (t_timers != nullptr &&
      t_timers_bytes >= static_cast<size_t>(plan.num_ctas) * 16 * sizeof(long long))
    params.timers = t_timers;
  // One past the last element of C the product may touch, in elements from C.
  params.out_span = (pm - 1) * ldc + pn;

  if (plan.stream_k) {
    const size_t need = plan.counters_bytes + plan.partials_bytes;
    char* ws = static_cast<char*>(workspace);
    if (ws != nullptr) {
      if (workspace_bytes < need || (reinterpret_cast<uintptr_t>(ws) & 255) != 0)
        return NEOGEMM_ERR_WORKSPACE;
    } else {
      std::lock_guard<std::mutex> lock(g_mu);
      rc = ensure_workspace(st, need, stream);
      if (rc != NEOGEMM_OK) return rc;
      ws = static_cast<char*>(st->workspace);
    }
    params.tile_counters = reinterpret_cast<int*>(ws);
    params.partials = reinterpret_cast<float*>(ws + plan.counters_bytes);
    // The last word of the counter region is the claim counter of the dynamic tail pool.
    params.counters_len = static_cast<long long>(plan.counters_bytes / sizeof(int)) - 1;
    params.partials_elems = static_cast<long long>(plan.partials_bytes / sizeof(float));
    params.dyn_counter = reinterpret_cast<int*>(ws) + params.counters_len;
  }

  t_last_store_path = tall_flip ? 2 : tall_tma ? 1 : 0;
  t_last_config[0] = plan.cta_group;
  t_last_config[1] = plan.block_n * plan.halves;
  t_last_config[2] = plan.kernel->stages;
  t_last_config[3] = plan.swap ? 1 : 0;
  t_last_config[4] = plan.stream_k ? 1 : 0;
  t_last_config[5] = plan.num_ctas;
  t_last_config[6] = plan.num_tiles;
  t_last_config[7] = plan.group_m;

  std::lock_guard<std::mutex> lock(g_mu);  // attr_done bookkeeping
  rc = launch(st, plan, mx, my, md, params, stream, t_override.tuning[10] != 0);
  if (rc == NEOGEMM_OK && plan.two_pass)
    rc = launch_reduce(st, plan, params, stream, t_override.tuning[10] != 0);
  return rc;
}

int ensure_copy_queues(DeviceState* st) {
  if (st->copy_in != nullptr) return NEOGEMM_OK;
  if (cudaStreamCreateWithFlags(&st->copy_in, cudaStreamNonBlocking) != cudaSuccess ||
      cudaStreamCreateWithFlags(&st->copy_out, cudaStreamNonBlocking) != cudaSuccess) {
    cudaGetLastError();
    st->copy_in = nullptr;
    return NEOGEMM_ERR_CUDA;
  }
  for (cudaEvent_t& e : st->copy_events) {
    if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) {
      cudaGetLastError();
      return NEOGEMM_ERR_CUDA;
    }
  }
  return NEOGEMM_OK;
}

int ensure_stage(DeviceState* st, int which, size_t bytes) {
  if (bytes <= st->stage_bytes[which]) return NEOGEMM_OK;
  if (st->stage[which] != nullptr) cudaFree(st->stage[which]);
  st->stage[which] = nullptr;
  st->stage_bytes[which] = 0;
  if (cudaMalloc(&st->stage[which], bytes) != cudaSuccess) {
    cudaGetLastError();
    return NEOGEMM_ERR_CUDA;
  }
  st->stage_bytes[which] = bytes;
  return NEOGEMM_OK;
}

}  // namespace
}  // namespace neogemm

using namespace neogemm;

extern "C" {

int neogemm_bf16_nt(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                    int64_t lda, int64_t ldb, int64_t ldc, int c_col_major, void* workspace,
                    size_t workspace_bytes, void* stream) {
  return gemm_device(A, B, C, M, N, K, lda, ldb, ldc, c_col_major, workspace, workspace_bytes,
                     static_cast<cudaStream_t>(stream));
}

int neogemm_bf16_nt_fused(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                          int64_t lda, int64_t ldb, int64_t ldc, int c_col_major, float alpha,
                          float beta, const void* bias, int activation, void* workspace,
                          size_t workspace_bytes, void* stream) {
  if (activation < 0 || activation > 2) return NEOGEMM_ERR_BAD_ARG;
  if (bias != nullptr && (reinterpret_cast<uintptr_t>(bias) & 1) != 0) return NEOGEMM_ERR_BAD_ARG;
  Fusion f;
  f.on = true;
  f.alpha = alpha;
  f.beta = beta;
  f.bias = bias;
  f.activation = activation;
  return gemm_device(A, B, C, M, N, K, lda, ldb, ldc, c_col_major, workspace, workspace_bytes,
                     static_cast<cudaStream_t>(stream), f);
}

int neogemm_bf16_nt_fused_f32(const void* A, const void* B, void* C, int64_t M, int64_t N,
                              int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int c_col_major,
                              float alpha, float beta, const void* bias, int activation,
                              void* workspace, size_t workspace_bytes, void* stream) {
  if (activation < 0 || activation > 2) return NEOGEMM_ERR_BAD_ARG;
  if (bias != nullptr && (reinterpret_cast<uintptr_t>(bias) & 1) != 0) return NEOGEMM_ERR_BAD_ARG;
  Fusion f;
  f.on = true;
  f.alpha = alpha;
  f.beta = beta;
  f.bias = bias;
  f.activation = activation;
  f.out_f32 = true;
  return gemm_device(A, B, C, M, N, K, lda, ldb, ldc, c_col_major, workspace, workspace_bytes,
                     static_cast<cudaStream_t>(stream), f);
}

size_t neogemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int c_col_major) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  int rc;
  int sm_count;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    DeviceState* st = device_state(&rc);
    if (st == nullptr) return 0;
    sm_count = st->sm_count;
  }
  Plan plan;
  const int64_t pm = c_col_major ? N : M;
  const int64_t pn = c_col_major ? M : N;
  // Unaligned C / pitch only ever selects the direct epilogue, whose needs are the larger.
  if (make_plan(pm, pn, K, 1, reinterpret_cast<const void*>(2), sm_count, t_override, &plan) !=
      NEOGEMM_OK)
    return 0;
  const size_t direct = plan.stream_k ? plan.counters_bytes + plan.partials_bytes : 0;
  if (make_plan(pm, pn, K, 8, nullptr, sm_count, t_override, &plan) != NEOGEMM_OK) return direct;
  const size_t aligned = plan.stream_k ? plan.counters_bytes + plan.partials_bytes : 0;
  return std::max(direct, aligned);
}

int neogemm_bf16_nt_host(const void* A_host, const void* B_host, void* C_host, int64_t M,
                         int64_t N, int64_t K, int c_col_major, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M < 0 || N < 0 || K < 0) return NEOGEMM_ERR_BAD_ARG;
  if (M == 0 || N == 0) return NEOGEMM_OK;
  if (C_host == nullptr || (K > 0 && (A_host == nullptr || B_host == nullptr)))
    return NEOGEMM_ERR_BAD_ARG;
  int rc;
  DeviceState* st;
  const size_t bytes_a = static_cast<size_t>(M) * K * 2, bytes_b = static_cast<size_t>(N) * K * 2,
               bytes_c = static_cast<size_t>(M) * N * 2;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    st = device_state(&rc);
    if (st == nullptr) return rc;
  }
  // The staging buffers, the two copy queues and their events are one set per device: a second
  // host thread calling in on the same device waits here until the first call has returned (the
  // call is synchronous anyway).
  std::lock_guard<std::mutex> one_call(st->host_entry_mu);
  {
    std::lock_guard<std::mutex> lock(g_mu);
    if ((rc = ensure_stage(st, 0, std::max<size_t>(bytes_a, 16))) != NEOGEMM_OK) return rc;
    if ((rc = ensure_stage(st, 1, std::max<size_t>(bytes_b, 16))) != NEOGEMM_OK) return rc;
    if ((rc = ensure_stage(st, 2, bytes_c)) != NEOGEMM_OK) return rc;
    if ((rc = ensure_copy_queues(st)) != NEOGEMM_OK) return rc;
  }
  // The rows of the matrix as stored ([M,N], or [N,M] for column-major C) come from one operand
  // (U); the other (V) is needed whole.  V goes up first; then U goes up in row chunks, each
  // chunk's product is launched as soon as it has landed, and its rows of C go back down while
  // the next chunk is still going up: the two PCIe directions and the GPU work overlap, so the
  // call takes about as long as the uploads alone.
  const int64_t pm = c_col_major ? N : M;
  const int64_t pn = c_col_major ? M : N;
  const char* U_host = static_cast<const char*>(c_col_major ? B_host : A_host);
  const char* V_host = static_cast<const char*>(c_col_major ? A_host : B_host);
  char* dU = static_cast<char*>(c_col_major ? st->stage[1] : st->stage[0]);
  char* dV = static_cast<char*>(c_col_major ? st->stage[0] : st->stage[1]);
  char* dC = static_cast<char*>(st->stage[2]);
  const size_t bytes_v = c_col_major ? bytes_a : bytes_b;
  int64_t chunks = std::min<int64_t>(kMaxHostChunks, std::max<int64_t>(1, pm / 512));
  if (K == 0) chunks = 1;
  const int64_t chunk_rows = ((pm + chunks - 1) / chunks + 255) / 256 * 256;

  auto fail = [&](int code) {
    cudaGetLastError();
    cudaStreamSynchronize(st->copy_in);
    cudaStreamSynchronize(st->copy_out);
    cudaStreamSynchronize(stream);
    cudaGetLastError();
    return code;
  };
  cudaEvent_t* ev = st->copy_events;
  // Everything below starts after the work already queued on the caller's stream.
  if (cudaEventRecord(ev[0], stream) != cudaSuccess ||
      cudaStreamWaitEvent(st->copy_in, ev[0], 0) != cudaSuccess ||
      cudaStreamWaitEvent(st->copy_out, ev[0], 0) != cudaSuccess)
    return fail(NEOGEMM_ERR_CUDA);
  if (K > 0) {
    if (cudaMemcpyAsync(dV, V_host, bytes_v, cudaMemcpyHostToDevice, st->copy_in) != cudaSuccess)
      return fail(NEOGEMM_ERR_CUDA);
  }
  // All uploads are queued before the first product or download.  Copies of both directions can
  // share one in-order hardware queue: a download that is still waiting for its product would
  // hold back every upload submitted after it, one product time per chunk (measured with a
  // sleeping kernel in place of the product: 5.45 -> 5.82 ms per call at 8 chunks).
  int64_t n_chunks = 0;
  for (int64_t r0 = 0; r0 < pm; r0 += chunk_rows, ++n_chunks) {
    const int64_t rows = std::min(chunk_rows, pm - r0);
    if (K > 0 &&
        cudaMemcpyAsync(dU + r0 * K * 2, U_host + r0 * K * 2, static_cast<size_t>(rows) * K * 2,
                        cudaMemcpyHostToDevice, st->copy_in) != cudaSuccess)
      return fail(NEOGEMM_ERR_CUDA);
    if (cudaEventRecord(ev[1 + 2 * n_chunks], st->copy_in) != cudaSuccess)
      return fail(NEOGEMM_ERR_CUDA);
  }
  int64_t index = 0;
  for (int64_t r0 = 0; r0 < pm; r0 += chunk_rows, ++index) {
    const int64_t rows = std::min(chunk_rows, pm - r0);
    cudaEvent_t up = ev[1 + 2 * index], done = ev[2 + 2 * index];
    if (cudaStreamWaitEvent(stream, up, 0) != cudaSuccess) return fail(NEOGEMM_ERR_CUDA);
    if (c_col_major)
      rc = gemm_device(dV, dU + r0 * K * 2, dC + r0 * pn * 2, M, rows, K, K, K, M, 1, nullptr, 0,
                       stream);
    else
      rc = gemm_device(dU + r0 * K * 2, dV, dC + r0 * pn * 2, rows, N, K, K, K, N, 0, nullptr, 0,
                       stream);
    if (rc != NEOGEMM_OK) return fail(rc);
    // A download starts on an upload boundary: besides its product it waits for the NEXT chunk's
    // upload to finish.  A download that starts in the middle of an upload costs that upload more
    // than the wait costs the download (measured, 16 chunks: 6.00 ms per call without this wait,
    // 5.49 ms with it; the same copies with no product in between take 5.40 ms).
    if (cudaEventRecord(done, stream) != cudaSuccess ||
        cudaStreamWaitEvent(st->copy_out, done, 0) != cudaSuccess ||
        (index + 1 < n_chunks &&
         cudaStreamWaitEvent(st->copy_out, ev[1 + 2 * (index + 1)], 0) != cudaSuccess) ||
        cudaMemcpyAsync(static_cast<char*>(C_host) + r0 * pn * 2, dC + r0 * pn * 2,
                        static_cast<size_t>(rows) * pn * 2, cudaMemcpyDeviceToHost,
                        st->copy_out) != cudaSuccess)
      return fail(NEOGEMM_ERR_CUDA);
  }
  if (cudaStreamSynchronize(st->copy_out) != cudaSuccess ||
      cudaStreamSynchronize(stream) != cudaSuccess) {
    cudaGetLastError();
    return NEOGEMM_ERR_CUDA;
  }
  if (st->status_host[0] != 0) return NEOGEMM_ERR_DEVICE_TIMEOUT;
  return NEOGEMM_OK;
}

int neogemm_device_status(int out[4]) {
  if (out == nullptr) return NEOGEMM_ERR_BAD_ARG;
  int rc;
  std::lock_guard<std::mutex> lock(g_mu);
  DeviceState* st = device_state(&rc);
  if (st == nullptr) return rc;
  for (int i = 0; i < 4; ++i) out[i] = st->status_host[i];
  return NEOGEMM_OK;
}

int neogemm_clear_device_status(void) {
  int rc;
  std::lock_guard<std::mutex> lock(g_mu);
  DeviceState* st = device_state(&rc);
  if (st == nullptr) return rc;
  if (cudaDeviceSynchronize() != cudaSuccess) {
    cudaGetLastError();
    return NEOGEMM_ERR_CUDA;
  }
  std::memset(st->status_host, 0, 64);
  // A launch that gave up may have left wave-pacing or stream-K arrival counters non-zero.
  if (st->pace_counters != nullptr &&
      cudaMemset(st->pace_counters, 0, kPaceSlots * 128) != cudaSuccess) {
    cudaGetLastError();
    return NEOGEMM_ERR_CUDA;
  }
  if (st->workspace != nullptr &&
      cudaMemset(st->workspace, 0, st->workspace_bytes) != cudaSuccess) {
    cudaGetLastError();
    return NEOGEMM_ERR_CUDA;
  }
  return NEOGEMM_OK;
}

const char* neogemm_status_str(int status) {
  switch (status) {
    case NEOGEMM_OK: return "ok";
    case NEOGEMM_ERR_BAD_ARG: return "bad argument (null pointer, negative size or short leading dimension)";
    case NEOGEMM_ERR_UNSUPPORTED: return "unsupported (K, lda, ldb must be multiples of 8; A, B 16-byte aligned; device must be sm_100)";
    case NEOGEMM_ERR_DESCRIPTOR: return "tensor-map encode failed or CUDA driver entry point unavailable";
    case NEOGEMM_ERR_LAUNCH: return "kernel launch failed";
    case NEOGEMM_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait expired in an earlier launch (see neogemm_device_status)";
    case NEOGEMM_ERR_WORKSPACE: return "workspace too small, misaligned or could not be allocated";
    case NEOGEMM_ERR_CUDA: return "CUDA runtime error";
    default: return "unknown status";
  }
}

int neogemm_last_config(int out[8]) {
  if (out == nullptr) return NEOGEMM_ERR_BAD_ARG;
  for (int i = 0; i < 8; ++i) out[i] = t_last_config[i];
  return NEOGEMM_OK;
}

int neogemm_last_store_path(void) { return t_last_store_path; }

int neogemm_set_override(int cta_group, int block_n, int swap, int stream_k, int group_m,
                         int max_ctas) {
  if (cta_group > 2 || cta_group == 0) return NEOGEMM_ERR_BAD_ARG;
  if (block_n > 0 && block_n != 16 && block_n != 32 && block_n != 64 && block_n != 128 &&
      block_n != 256)
    return NEOGEMM_ERR_BAD_ARG;
  t_override.cta_group = cta_group;
  t_override.block_n = block_n;
  t_override.swap = swap;
  t_override.stream_k = stream_k;
  t_override.group_m = group_m;
  t_override.max_ctas = max_ctas;
  return NEOGEMM_OK;
}

int neogemm_set_phase_timers(void* device_buffer, size_t bytes) {
  if (device_buffer != nullptr && (reinterpret_cast<uintptr_t>(device_buffer) & 7) != 0)
    return NEOGEMM_ERR_BAD_ARG;
  t_timers = static_cast<long long*>(device_buffer);
  t_timers_bytes = device_buffer ? bytes : 0;
  return NEOGEMM_OK;
}

int neogemm_set_tuning(int key, int value) {
  if (key < 0 || key > 12 || (key == 6 && (value == 0 || value > 3)) || (key >= 8 && value > 1) || (key == 7 && value > 4) || (key == 5 && value > 3) || value > 1000000 || (key == 0 && value > 31) || (key == 3 && value > 1) ||
      (key == 4 && value > 4))
    return NEOGEMM_ERR_BAD_ARG;
  t_override.tuning[key] = value;
  return NEOGEMM_OK;
}

int neogemm_debug_wait_expiry(unsigned int limit_us, unsigned long long* waited_ns_out) {
  if (limit_us == 0 || limit_us > 100000) return NEOGEMM_ERR_BAD_ARG;   // 0.1 s at most
  int rc;
  DeviceState* st;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    st = device_state(&rc);
  }
  if (st == nullptr) return rc;
  if (st->status_host[0] != 0) return NEOGEMM_ERR_DEVICE_TIMEOUT;
  // The waited time comes back through the same mapped page as the status record (words 8..9).
  unsigned long long* waited_host = reinterpret_cast<unsigned long long*>(st->status_host + 8);
  unsigned long long* waited_dev = reinterpret_cast<unsigned long long*>(st->status_dev + 8);
  *waited_host = 0;
  GemmParams params;
  std::memset(&params, 0, sizeof(params));
  params.status = st->status_dev;
  wait_expiry_selftest_kernel<<<1, 32>>>(params, static_cast<unsigned long long>(limit_us) * 1000ull,
                                         waited_dev);
  if (cudaGetLastError() != cudaSuccess) return NEOGEMM_ERR_LAUNCH;
  if (cudaDeviceSynchronize() != cudaSuccess) {
    cudaGetLastError();
    return NEOGEMM_ERR_CUDA;
  }
  if (waited_ns_out != nullptr) *waited_ns_out = *waited_host;
  return NEOGEMM_OK;
}

int neogemm_version(void) { return 100; }

int neogemm_debug_plan(int64_t M, int64_t N, int64_t K, int64_t ldc, int c_col_major, int sm_count,
                       int* plan_out, int* segments, int max_segments) {
  if (plan_out == nullptr || M <= 0 || N <= 0 || K <= 0 || sm_count <= 0)
    return -NEOGEMM_ERR_BAD_ARG;
  Plan plan;
  const int64_t pm = c_col_major ? N : M;
  const int64_t pn = c_col_major ? M : N;
  const int rc = make_plan(pm, pn, K, ldc, nullptr, sm_count, t_override, &plan);
  if (rc != NEOGEMM_OK) return -rc;
  const int fields[16] = {plan.cta_group, plan.block_n * plan.halves, plan.kernel->stages, plan.swap ? 1 : 0,
                          plan.stream_k ? 1 : 0, plan.num_ctas, plan.num_tiles, plan.group_m,
                          plan.epi, plan.Md, plan.Nd, plan.num_m_tiles, plan.num_n_tiles,
                          plan.num_k_blocks, plan.max_contrib, plan.sk_first_tile};
  for (int i = 0; i < 16; ++i) plan_out[i] = fields[i];
  GemmParams params;
  std::memset(&params, 0, sizeof(params));
  params.num_m_tiles = plan.num_m_tiles;
  params.num_n_tiles = plan.num_n_tiles;
  params.num_tiles = plan.num_tiles;
  params.num_k_blocks = plan.num_k_blocks;
  params.group_m = plan.group_m;
  params.stream_k = plan.stream_k ? 1 : 0;
  params.sk_first_tile = plan.sk_first_tile;
  params.sk_splits = plan.sk_splits;
  params.dyn_pieces = plan.dyn_pieces;
  params.dyn_ppt = plan.dyn_ppt;
  params.dyn_piece_kb = plan.dyn_piece_kb;
  params.dyn_static_kb = plan.dyn_static_kb;
  const int workers = plan.num_ctas / plan.cta_group;
  int count = 0;
  for (int w = 0; w < workers; ++w) {
    SegmentIter it(params, w, workers);
    Segment seg;
    while (it.next(seg)) {
      if (segments != nullptr && count < max_segments) {
        int tm, tn;
        tile_coords(params, seg.tile, tm, tn);
        int* o = segments + 8 * count;
        o[0] = w; o[1] = seg.tile; o[2] = seg.kb_begin; o[3] = seg.kb_count;
        o[4] = seg.contrib; o[5] = seg.n_contrib; o[6] = tm; o[7] = tn;
      }
      ++count;
    }
  }
  // Pieces of the dynamic tail pool: who computes them is decided at run time; they are listed
  // with the worker that would take them if claims came round-robin.
  if (plan.dyn_pieces > 0) {
    SegmentIter it(params, 0, workers);
    for (int id = 0; id < plan.dyn_pieces; ++id) {
      Segment seg;
      it.piece(seg, id);
      if (segments != nullptr && count < max_segments) {
        int tm, tn;
        tile_coords(params, seg.tile, tm, tn);
        int* o = segments + 8 * count;
        o[0] = id % workers; o[1] = seg.tile; o[2] = seg.kb_begin; o[3] = seg.kb_count;
        o[4] = seg.contrib; o[5] = seg.n_contrib; o[6] = tm; o[7] = tn;
      }
      ++count;
    }
  }
  return count;
}


// ------------------------------------------------------------------------------------------
// Entry point that allocates nothing.
//
// Who needs it: code that must not (or cannot) ask the CUDA allocator for memory at the moment
// it multiplies - a serving loop whose memory pool already owns the whole device, a real-time
// path where an allocation's latency or failure is unacceptable, a plugin that is forbidden to
// touch the process's allocator.  neogemm_bf16_nt() may allocate on its first call per device
// (a pinned status word) and whenever a skinny shape needs a larger library-owned stream-K
// workspace; this variant never does.  Its stream-K scratch is the fixed array below, which
// every GPU that loads the library carries until the process exits.
//
// What "nothing" covers: no call below reaches cudaMalloc, cudaFree, cudaHostAlloc or an
// allocating library routine.  What it cannot cover is the CUDA driver's own lazy loading: the
// first use of the library's code on a device makes the driver place the module (the 32 MiB array
// and the kernels) in device memory.  neogemm_noalloc_init() forces all of that to happen at a
// moment the caller chooses - before its pool takes the device.
// ------------------------------------------------------------------------------------------
namespace {

constexpr size_t kStaticScratchBytes = 32u << 20;   // 32 MiB: counters (256 KiB) + partials
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
static __device__ __align__(16) int g_static_status[4];

struct StaticState {
  bool ready = false;                 // set only once the whole set-up has succeeded
  bool warmed = false;                // every kernel variant loaded and configured
  unsigned char* scratch = nullptr;   // DEVICE address of g_static_scratch on this device
  int* status = nullptr;              // DEVICE address of g_static_status on this device
  int seen[4] = {0, 0, 0, 0};         // the device status word as the host last read it
  DeviceState launch_state;           // only sm_count and the per-kernel attribute flags are used
};
StaticState g_static[kMaxDevices];
PFN_cuTensorMapEncodeTiled_v12000 g_static_encode = nullptr;

// In host code the names g_static_scratch / g_static_status are host-side stand-ins, not device
// addresses; the addresses a kernel may use come from cudaGetSymbolAddress, once per device,
// with that device current.  Called with g_mu held.  A failed attempt is not remembered: a
// transient error (the device had no room for the module at that moment) can be retried.
StaticState* static_state(int* code) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    cudaGetLastError();
    *code = NEOGEMM_ERR_UNSUPPORTED;
    return nullptr;
  }
  StaticState& st = g_static[dev];
  if (st.ready) {
    *code = NEOGEMM_OK;
    return &st;
  }
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
      major != 10 ||
      cudaDeviceGetAttribute(&st.launch_state.sm_count, cudaDevAttrMultiProcessorCount, dev) !=
          cudaSuccess) {
    cudaGetLastError();
    *code = NEOGEMM_ERR_UNSUPPORTED;
    return nullptr;
  }
  if (g_static_encode == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) ==
            cudaSuccess && q == cudaDriverEntryPointSuccess) {
      g_static_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
    } else {
      cudaGetLastError();
      *code = NEOGEMM_ERR_DESCRIPTOR;
      return nullptr;
    }
  }
  void* scratch = nullptr;
  void* status = nullptr;
  if (cudaGetSymbolAddress(&scratch, g_static_scratch) != cudaSuccess ||
      cudaGetSymbolAddress(&status, g_static_status) != cudaSuccess || scratch == nullptr ||
      status == nullptr) {
    cudaGetLastError();
    *code = NEOGEMM_ERR_CUDA;
    return nullptr;
  }
  st.scratch = static_cast<unsigned char*>(scratch);
  st.status = static_cast<int*>(status);
  st.ready = true;
  *code = NEOGEMM_OK;
  return &st;
}

// Same geometry as get_tensor_map(), encoded straight into the caller's variable: no cache, so no
// host heap growth either.
int encode_map_uncached(const void* base, uint64_t inner, uint64_t rows, uint64_t pitch_bytes,
                        uint32_t box_rows, int for_store, CUtensorMap* out) {
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (pitch_bytes & 15) != 0 ||
      pitch_bytes >= (1ull << 40) || inner == 0 || rows == 0 || inner > 0xffffffffull ||
      rows > 0xffffffffull || box_rows == 0 || box_rows > 256) {
    return NEOGEMM_ERR_UNSUPPORTED;
  }
  cuuint64_t dims[2] = {inner, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {for_store >= 1000 ? static_cast<cuuint32_t>(for_store - 1000) : 64u, box_rows};
  if (for_store >= 1000 && (for_store > 1256 || (for_store & 7) != 0)) return NEOGEMM_ERR_UNSUPPORTED;
  cuuint32_t elem_strides[2] = {1, 1};
  const CUresult r = g_static_encode(
      out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
      elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
      for_store >= 1000 ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B,
      for_store ? CU_TENSOR_MAP_L2_PROMOTION_NONE : CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? NEOGEMM_OK : NEOGEMM_ERR_DESCRIPTOR;
}

}  // namespace

int neogemm_noalloc_init(void) {
  std::lock_guard<std::mutex> lock(g_mu);
  int rc;
  StaticState* st = static_state(&rc);
  if (st == nullptr) return rc;
  if (st->warmed) return NEOGEMM_OK;
  // Configuring a kernel makes the driver load it: after this loop no shape can meet a variant
  // that still has to be placed on the device.
  int n;
  const KernelEntry* table = kernel_table(&n);
  for (int i = 0; i < n; ++i) {
    if (st->launch_state.attr_done[i]) continue;
    if (cudaFuncSetAttribute(table[i].fn, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             table[i].smem_bytes) != cudaSuccess) {
      cudaGetLastError();
      return NEOGEMM_ERR_LAUNCH;
    }
    st->launch_state.attr_done[i] = true;
  }
  cudaFuncAttributes unused;
  if (cudaFuncGetAttributes(&unused, reinterpret_cast<const void*>(
                                         &wait_expiry_selftest_kernel)) != cudaSuccess) {
    cudaGetLastError();
    return NEOGEMM_ERR_LAUNCH;
  }
  if (cudaMemset(st->status, 0, sizeof(int) * 4) != cudaSuccess) {
    cudaGetLastError();
    return NEOGEMM_ERR_CUDA;
  }
  st->warmed = true;
  return NEOGEMM_OK;
}

int neogemm_noalloc_status(int out[4], void* stream_) {
  if (out == nullptr) return NEOGEMM_ERR_BAD_ARG;
  std::lock_guard<std::mutex> lock(g_mu);
  int rc;
  StaticState* st = static_state(&rc);
  if (st == nullptr) return rc;
  // The word lives in device memory: wait for the caller's launches, then copy 16 bytes into the
  // caller's array.  Nothing is allocated; the copy is synchronous.
  int word[4] = {0, 0, 0, 0};
  if (cudaStreamSynchronize(static_cast<cudaStream_t>(stream_)) != cudaSuccess ||
      cudaMemcpy(word, st->status, sizeof(word), cudaMemcpyDeviceToHost) != cudaSuccess) {
    cudaGetLastError();
    return NEOGEMM_ERR_CUDA;
  }
  for (int i = 0; i < 4; ++i) out[i] = st->seen[i] = word[i];
  return NEOGEMM_OK;
}

int neogemm_noalloc_clear_status(void) {
  std::lock_guard<std::mutex> lock(g_mu);
  int rc;
  StaticState* st = static_state(&rc);
  if (st == nullptr) return rc;
  // A launch that gave up may also have left arrival counters of the fixed scratch non-zero;
  // every call clears those before it launches, so only the status word needs attention here.
  if (cudaDeviceSynchronize() != cudaSuccess ||
      cudaMemset(st->status, 0, sizeof(int) * 4) != cudaSuccess) {
    cudaGetLastError();
    return NEOGEMM_ERR_CUDA;
  }
  for (int i = 0; i < 4; ++i) st->seen[i] = 0;
  return NEOGEMM_OK;
}

int neogemm_debug_wait_expiry_noalloc(unsigned int limit_us) {
  if (limit_us == 0 || limit_us > 100000) return NEOGEMM_ERR_BAD_ARG;
  std::lock_guard<std::mutex> lock(g_mu);
  int rc;
  StaticState* st = static_state(&rc);
  if (st == nullptr) return rc;
  GemmParams params;
  std::memset(&params, 0, sizeof(params));
  params.status = st->status;
  wait_expiry_selftest_kernel<<<1, 32>>>(params, static_cast<unsigned long long>(limit_us) * 1000ull,
                                         nullptr);
  if (cudaGetLastError() != cudaSuccess) return NEOGEMM_ERR_LAUNCH;
  if (cudaDeviceSynchronize() != cudaSuccess) {
    cudaGetLastError();
    return NEOGEMM_ERR_CUDA;
  }
  return NEOGEMM_OK;
}

int neogemm_bf16_nt_noalloc(const void* A, const void* B, void* C, int64_t M, int64_t N,
                            int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int c_col_major,
                            void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int rc = validate(A, B, C, M, N, K, lda, ldb, ldc, c_col_major);
  if (rc != NEOGEMM_OK) return rc;
  if (M == 0 || N == 0) return NEOGEMM_OK;

  std::lock_guard<std::mutex> lock(g_mu);
  StaticState* st = static_state(&rc);
  if (st == nullptr) return rc;
  // An error a launch of this entry point recorded on the device, as last read back by
  // neogemm_noalloc_status(): refuse until neogemm_noalloc_clear_status().
  if (st->seen[0] != 0) return NEOGEMM_ERR_DEVICE_TIMEOUT;

  const int64_t pm = c_col_major ? N : M;
  const int64_t pn = c_col_major ? M : N;
  if (K == 0) {
    if (cudaMemset2DAsync(C, static_cast<size_t>(ldc) * 2, 0, static_cast<size_t>(pn) * 2,
                          static_cast<size_t>(pm), stream) != cudaSuccess) {
      cudaGetLastError();
      return NEOGEMM_ERR_CUDA;
    }
    return NEOGEMM_OK;
  }
  const void* U = c_col_major ? B : A;
  const void* V = c_col_major ? A : B;
  const int64_t ldu = c_col_major ? ldb : lda;
  const int64_t ldv = c_col_major ? lda : ldb;

  Plan plan;
  const Override no_override;
  // Only the skinny (direct-store) kernels take scratch here: the cut last wave of the large
  // kernels is left off, so that large shapes never depend on the fixed array's size.
  rc = make_plan(pm, pn, K, ldc, C, st->launch_state.sm_count, no_override, &plan, false, true);
  if (rc != NEOGEMM_OK) return rc;
  if (plan.stream_k && plan.counters_bytes + plan.partials_bytes > kStaticScratchBytes)
    return NEOGEMM_ERR_WORKSPACE;   // beyond the fixed scratch: use neogemm_bf16_nt()

  const void* X = plan.swap ? V : U;
  const void* Y = plan.swap ? U : V;
  const int64_t ldx = plan.swap ? ldv : ldu;
  const int64_t ldy = plan.swap ? ldu : ldv;
  CUtensorMap mx, my, md;
  std::memset(&md, 0, sizeof(md));
  rc = encode_map_uncached(X, static_cast<uint64_t>(K), static_cast<uint64_t>(plan.Md),
                           static_cast<uint64_t>(ldx) * 2,
                           plan.mhalves == 2 ? static_cast<uint32_t>(plan.tile_rows) : 128u, 0, &mx);
  if (rc != NEOGEMM_OK) return rc;
  rc = encode_map_uncached(Y, static_cast<uint64_t>(K), static_cast<uint64_t>(plan.Nd),
                           static_cast<uint64_t>(ldy) * 2,
                           static_cast<uint32_t>(plan.block_n / plan.cta_group), 0, &my);
  if (rc != NEOGEMM_OK) return rc;
  if (plan.epi == kEpiTmaStore) {
    rc = encode_map_uncached(C, static_cast<uint64_t>(plan.Nd), static_cast<uint64_t>(plan.Md),
                             static_cast<uint64_t>(ldc) * 2, 32, 1, &md);
    if (rc != NEOGEMM_OK) return rc;
  }
  bool tall_tma = tall_tile_tma_store(plan, C, ldc, 2);
  bool tall_flip = tall_tma && plan.cta_group == 2 && plan.block_n == 128;
  if (tall_tma) {
    rc = encode_map_uncached(C, static_cast<uint64_t>(plan.Md), static_cast<uint64_t>(plan.Nd),
                             static_cast<uint64_t>(ldc) * 2,
                             tall_flip ? 32u : static_cast<uint32_t>(plan.block_n),
                             1000 + plan.tile_rows, &md);
    if (rc != NEOGEMM_OK) tall_tma = tall_flip = false;   // stores from registers serve any C
  }

  GemmParams params;
  std::memset(&params, 0, sizeof(params));
  params.Md = plan.Md;
  params.Nd = plan.Nd;
  params.K = static_cast<int>(K);
  params.num_m_tiles = plan.num_m_tiles;
  params.num_n_tiles = plan.num_n_tiles;
  params.num_tiles = plan.num_tiles;
  params.num_k_blocks = plan.num_k_blocks;
  params.group_m = plan.group_m;
  params.tile_rows = plan.tile_rows;
  params.l2_hints = ((plan.epi == kEpiDirect && plan.num_n_tiles == 1) ? 24 : kDefaultTuning[0]) |
                    (tall_flip ? 64 : tall_tma ? 32 : 0);
  params.epi_wait_hint_ns = kDefaultTuning[1];
  params.main_wait_hint_ns = kDefaultTuning[2];
  params.wide_prologue = kDefaultWidePrologue;
  params.out = static_cast<__nv_bfloat16*>(C);
  params.out_stride_r = plan.swap ? 1 : ldc;
  params.out_stride_c = plan.swap ? ldc : 1;
  params.out_span = (pm - 1) * ldc + pn;
  params.stream_k = plan.stream_k ? 1 : 0;
  params.sk_first_tile = plan.sk_first_tile;
  params.sk_splits = plan.sk_splits;
  params.dyn_pieces = plan.dyn_pieces;
  params.dyn_ppt = plan.dyn_ppt;
  params.dyn_piece_kb = plan.dyn_piece_kb;
  params.dyn_static_kb = plan.dyn_static_kb;
  params.max_contrib = plan.max_contrib;
  params.sk_two_pass = plan.two_pass ? 1 : 0;
  params.status = st->status;
  params.timers = nullptr;
  // Same K-direction rule as the regular entry point, so that both give the same bits.
  params.k_alternate = (kDefaultKAlternate && !plan.stream_k && plan.epi == kEpiTmaStore &&
                        plan.num_tiles > plan.num_ctas / plan.cta_group) ? 1 : 0;
  if (plan.stream_k) {
    // Every call shares the array and it keeps the previous call's contents: the arrival
    // counters must start at zero, so clear their region in stream order before the launch.
    if (cudaMemsetAsync(st->scratch, 0, plan.counters_bytes, stream) != cudaSuccess) {
      cudaGetLastError();
      return NEOGEMM_ERR_CUDA;
    }
    params.tile_counters = reinterpret_cast<int*>(st->scratch);
    params.partials = reinterpret_cast<float*>(st->scratch + plan.counters_bytes);
    params.counters_len = static_cast<long long>(plan.counters_bytes / sizeof(int)) - 1;
    params.partials_elems = static_cast<long long>(plan.partials_bytes / sizeof(float));
    params.dyn_counter = reinterpret_cast<int*>(st->scratch) + params.counters_len;
  }
  t_last_store_path = tall_flip ? 2 : tall_tma ? 1 : 0;
  t_last_config[0] = plan.cta_group;
  t_last_config[1] = plan.block_n * plan.halves;
  t_last_config[2] = plan.kernel->stages;
  t_last_config[3] = plan.swap ? 1 : 0;
  t_last_config[4] = plan.stream_k ? 1 : 0;
  t_last_config[5] = plan.num_ctas;
  t_last_config[6] = plan.num_tiles;
  t_last_config[7] = plan.group_m;
  rc = launch(&st->launch_state, plan, mx, my, md, params, stream);
  if (rc == NEOGEMM_OK && plan.two_pass) rc = launch_reduce(&st->launch_state, plan, params, stream);
  return rc;
}

}  // extern "C"
