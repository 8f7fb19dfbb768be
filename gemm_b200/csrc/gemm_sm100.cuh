// Persistent, warp-specialised BF16 GEMM for sm_100a:  D[Md,Nd] = X[Md,K] * Y[Nd,K]^T,
// X and Y K-major bf16, fp32 accumulation in tensor memory, bf16 (round-to-nearest-even) result.
//
// It computes what the reference's gemmkernel computes per 64x64 tile with wgmma
// (neogemmV02.cu:179-260) and what its tcgen05 sketches intended (nemgemmV03.cu:208-341), but is
// organised for Blackwell:
//   warp 0      TMA producer: one lane streams 128B-swizzled K-major boxes of X and Y into a
//               kStages-deep shared-memory ring, signalling full[] mbarriers by byte count;
//   warp 1      UMMA issuer: one lane (of the leader CTA when two CTAs share a tile) issues
//               tcgen05.mma into one of two TMEM accumulators and releases ring slots / publishes
//               finished accumulators with tcgen05.commit;
//   warps 2-5   epilogue: tcgen05.ld -> bf16 -> swizzled shared staging -> TMA store (or direct
//               strided global stores), overlapped with the next tile's main loop through the
//               second accumulator.
// With kCtaGroup == 2 a cluster of two CTAs computes a (256 x BLOCK_N) tile: each CTA loads its
// own 128 rows of X and its own half of the Y tile (plain per-CTA TMA loads whose byte counts
// are credited to the leader's barrier), and the leader's MMA reads both halves.
//
// Work is handed out as segments (tile, first k-block, k-block count).  In the data-parallel
// schedule every segment is a whole tile.  In the stream-K schedule (skinny, HBM-bound shapes) the
// (tile x k-block) space is cut into equal contiguous ranges, one per CTA, so every SM streams the
// same number of bytes; tiles cut by a range boundary are finished by whichever contributor
// arrives last, which sums the fp32 partials in a fixed order.
//
// Every mbarrier wait is bounded (ptx::mbar_wait).  On expiry the role records a code in
// `params.status`, raises the CTA's abort flag and falls through to the common tear-down, which
// lets copies in flight land and frees tensor memory.  The kernel never traps or spins forever.
#pragma once

#include "ptx.cuh"

namespace neogemm {

enum EpilogueMode : int {
  kEpiTmaStore = 0,  // row-major D, 16-byte-aligned pitch: staged through swizzled smem + TMA store
  kEpiDirect = 1,    // arbitrary (row, col) strides straight from registers, bounds-checked
};

// Device-side error codes written to the status word (first error wins).
enum DeviceError : int {
  kDevOk = 0,
  kDevTimeoutProducer = 1,   // TMA warp gave up waiting for a free ring slot
  kDevTimeoutMmaFull = 2,    // MMA warp gave up waiting for operand bytes
  kDevTimeoutMmaTmem = 3,    // MMA warp gave up waiting for a drained accumulator
  kDevTimeoutEpilogue = 4,   // epilogue gave up waiting for a finished accumulator
  kDevTmemAddress = 5,       // tensor-memory allocation did not start at column 0 (pair mode)
  kDevBounds = 6,            // an index left its buffer (access skipped); aux: 1 partials, 2 counters, 3 C
  kDevTimeoutScheduler = 7,  // a role gave up waiting on the dynamic-claim queue
};

struct GemmParams {
  int Md, Nd, K;
  int num_m_tiles, num_n_tiles, num_tiles, num_k_blocks;
  int group_m;               // tile rows per raster group (L2 reuse)
  int tile_rows;             // tall-tile kernels: rows of X per tile (a multiple of 8 between 129
                             // and kTallRows, chosen so that the tiles spread evenly over the
                             // SMs); 0 for every other kernel, whose tile height is fixed
  int l2_hints;              // bit 0: X loads evict-last, bit 1: Y loads evict-first,
                             // bit 2: D stores evict-first, bit 3: X loads evict-first,
                             // bit 4: Y loads evict-last (0 = no hints)
                             // bit 5 (set by the launcher, not a hint): a tall tile stores its
                             // transposed bf16 result through the TMA unit, tmap_d is its map
                             // bit 6 (set by the launcher): the same with the operands' roles
                             // exchanged in the MMA (GemmConfig::kFlippable)
  int epi_wait_hint_ns;      // suspend hint of the epilogue's wait for an accumulator (0 = none)
  int main_wait_hint_ns;     // suspend hint of the producer's and the MMA warp's ring waits
  int wide_prologue;         // two-half tiles: k-blocks issued for half 0 alone at a tile's start
  // Wave pacing (plain round-robin schedules of many waves): an arrival counter in global
  // memory, zero between launches, and how long a worker may wait at a wave's start for the
  // others to arrive.  Null = off.
  int* pace_counter;
  int pace_timeout_ns;
  // Whole tiles of odd waves walk K backwards: the k-slices of the row panel a worker group used
  // last in one wave are the first ones the next wave asks for, while L2 still holds them.
  int k_alternate;
  // Direct epilogue / split partials.
  __nv_bfloat16* out;
  // fp32 result (fused entry point only): when non-null the epilogue writes the unrounded fp32
  // values here instead of bf16 to `out`, with the same strides (in elements), and reads the
  // beta term from c_in32.  Two-half tiles do not take this path (the launcher never picks them
  // for an fp32 result).
  float* out32;
  const float* c_in32;
  long long out_stride_r, out_stride_c;
  // Stream-K (zero / null in the data-parallel schedule).
  int stream_k;              // 1: tiles >= sk_first_tile are cut: CTA c owns units [c*U/G, (c+1)*U/G)
                             // of their (tile x k-block) space; tiles below go round-robin
  int sk_first_tile;         // first tile of the stream-K region (0 = every tile)
  int sk_splits;             // > 0: every tile of the region is cut into this many equal k-chunks,
                             // one per worker (worker w takes chunk w / tiles of tile w % tiles),
                             // instead of one contiguous unit range per worker
  int max_contrib;           // partial slots per tile in `partials`
  // Dynamic tail pool (pure stream-K only; all zero otherwise).  The last dyn_ppt * dyn_piece_kb
  // k-blocks of every tile are not part of any CTA's static range: they form dyn_pieces fixed
  // pieces that CTAs claim from `dyn_counter` as they run out of static work, which evens out
  // the uneven HBM service the SMs get.  Pieces are fixed (tile, k-range) units with their own
  // partial slot, so the result does not depend on who computed which piece.
  int dyn_pieces, dyn_ppt, dyn_piece_kb, dyn_static_kb;
  int* dyn_counter;          // zero before launch; the launch's last claim re-zeroes it
  float* partials;           // [stream-K tiles][max_contrib][BLOCK_N][TILE_M] fp32
  int* tile_counters;        // [stream-K tiles][kCtaGroup][4], zero before launch; the last arriver
                             // of each entry re-zeroes it
  // Fused epilogue  D = act(alpha * (X Y^T) + beta * C_in + bias)  (all off: fuse == 0).
  // The reference declares alpha/beta kernel parameters but never uses them (neogemmv4.cu:166).
  int fuse;                  // 0: plain store; 1: apply the fields below
  float alpha, beta;
  const __nv_bfloat16* c_in; // read with the strides of `out` when beta != 0 (may alias `out`)
  const __nv_bfloat16* bias; // null, or one bf16 per output column of C = A B^T (length N)
  int bias_on_rows;          // 1: the bias index runs along the rows of D, 0: along its columns
  int activation;            // 0 none, 1 ReLU, 2 GELU (tanh form)
  // Extents for the self-checks of every global access the kernel computes itself.
  long long partials_elems, counters_len, out_span;
  // Optional phase timers (null in production): 16 int64 per CTA, see PhaseTimer below.
  long long* timers;
  // Error reporting: status[0] = code, [1] = blockIdx, [2] = segment index, [3] = stage / acc.
  int* status;
  int sk_two_pass;           // 1: contributors of a cut tile only publish their partials; the
                             // closing sums, the epilogue arithmetic and the stores of those
                             // tiles are done by splitk_reduce_kernel, launched right behind
                             // this kernel.  0: the last contributor to arrive finishes the tile.
};

template <int kCtaGroup_, int BLOCK_N_, int kStages_, int kEpiMode_, int kNHalves_ = 1,
          int kMHalves_ = 1>
struct GemmConfig {
  // kMHalves == 2 ("tall tile"): a CTA's tile is up to kTallRows rows of X - one 128-row block
  // and a second, partly filled one below it - that share the Y operand, each block with its own
  // TMEM accumulator.  Made for the skinny, HBM-bound shapes: the tile height is a run-time value
  // (GemmParams::tile_rows) picked so that the rows of X spread evenly over all SMs (28672 rows on
  // 148 SMs: 200 rows each on 144 of them, instead of 128-row tiles two to some SMs and one to
  // others), Y enters an SM once per tile instead of once per 128 rows, and one CTA per SM leaves
  // room for a deep ring of the streamed operand.  The second MMA block always spans 128 rows of
  // shared memory; rows past the tile's height hold stale bytes, their accumulator lanes are
  // never stored.  Whole tiles only (no stream-K), direct-store epilogue.  With kCtaGroup == 2 two
  // such CTAs share Y as well: each loads half of its rows, the pair's MMA reads both halves, so Y
  // takes half as much of every ring slot and the ring of the streamed operand gets deeper.
  static constexpr int kMHalves = kMHalves_;
  static constexpr int kTallRows = 208;
  // A pair of tall tiles with 128 columns can run with the operands' roles exchanged in the MMA
  // (a run-time choice, GemmParams::l2_hints bit 6).  As described above the pair issues two
  // 256 x 128 instructions per k-step, the second for rows 128..255 of each CTA's tile of which
  // only tile_rows - 128 exist: at 200 rows 22 % of the tensor work is spent on rows nobody
  // stores, and under the power cap, where these shapes run at half the idle clock, the tensor
  // pipe is the busiest unit of the SM.  Exchanged, the 2 x 64 rows of Y are the M side of a
  // 128-row pair instruction and X's rows are its N side, which comes in steps of 16: one
  // instruction of N = 256 (rows 0..127 of both CTAs' tiles) and one of N = 2 x (tile_rows -
  // 128), nothing wasted.  The same bytes sit in the same shared memory; only the descriptors
  // trade places.  The accumulator then is D transposed: lane l of a CTA holds row
  // 64 x rank + (l mod 64) of Y against tile row j of the CTA l / 64 of the pair in column j.
  static constexpr bool kFlippable = (kMHalves_ == 2 && kCtaGroup_ == 2 && BLOCK_N_ == 128);
  static constexpr int kCtaGroup = kCtaGroup_;
  static constexpr int BLOCK_N = BLOCK_N_;           // UMMA N
  // kNHalves == 2: the tile is two UMMA-N-wide halves side by side that share the X operand, each
  // with its own TMEM accumulator (all 512 columns in use, so there is no second accumulator set:
  // the next tile's main loop waits half by half for the epilogue to drain).  The point is fewer
  // bytes into the SM per flop: X is fetched once for 2 x BLOCK_N columns.
  static constexpr int kNHalves = kNHalves_;
  static constexpr int TILE_N = BLOCK_N * kNHalves;  // tile columns
  static constexpr int kStages = kStages_;
  static constexpr int kEpiMode = kEpiMode_;
  static constexpr int BLOCK_M = 128;                 // rows of X (TMEM lanes) per CTA
  static constexpr int UMMA_M = BLOCK_M * kCtaGroup;
  static constexpr int TILE_M = UMMA_M * kMHalves;    // rows of X per tile
  static constexpr int BLOCK_K = 64;                  // 64 bf16 = one 128-byte swizzle row
  static constexpr int UMMA_K = 16;
  static constexpr int LOAD_N = BLOCK_N / kCtaGroup;  // rows of Y each CTA fetches
  static constexpr int SMEM_X_HALF = BLOCK_M * BLOCK_K * 2;
  static constexpr int SMEM_X = (kMHalves == 2) ? kTallRows * BLOCK_K * 2 : SMEM_X_HALF;
  static constexpr int SMEM_Y_HALF = LOAD_N * BLOCK_K * 2;
  static constexpr int SMEM_Y = kNHalves * SMEM_Y_HALF;
  static constexpr int SMEM_STAGE = SMEM_X + SMEM_Y;
  static constexpr int EPI_COLS = 64;                 // columns per TMA-store box (128 B of bf16)
  static constexpr int SMEM_EPI_WARP_BUF = 32 * EPI_COLS * 2;  // 4 KB: 32 rows x 128 B
  // One-half tiles: four epilogue warps, two staging buffers each.  Two-half tiles: eight
  // epilogue warps (four per half, so both halves drain at once), one buffer each.
  static constexpr int kEpiWarps = 4 * kNHalves;
  static constexpr int kEpiBufs = (kNHalves == 1) ? 2 : 1;
  // Direct mode works through the accumulator kDirectCols columns at a time and stages each such
  // step of a warp's 32 rows transposed ([column][32 rows], 64 B per column) so that a transposed
  // result leaves as 16-byte vectors instead of 2-byte scalars.
  static constexpr int kDirectCols = (BLOCK_N >= 32) ? 32 : 16;
  static constexpr int SMEM_EPI_T_WARP = kDirectCols * 64;
  // A tall tile is its CTA's only tile and stages in the operand ring, which is idle by then.
  // What it needs behind the ring instead is room for its second MMA block to read: that block
  // always spans rows 128..255 of a slot's X region, i.e. bytes up to 2 x SMEM_X_HALF from the
  // slot's start, which for narrow tiles is more than a slot - past the LAST slot that would be
  // past the CTA's shared memory, an illegal address.  (What is read there feeds accumulator
  // lanes that are never stored.)
  static constexpr int SMEM_TALL_PAD =
      (kMHalves == 2 && 2 * SMEM_X_HALF > SMEM_STAGE) ? 2 * SMEM_X_HALF - SMEM_STAGE : 0;
  static constexpr int SMEM_EPI = (kEpiMode == kEpiTmaStore) ? kEpiWarps * kEpiBufs * SMEM_EPI_WARP_BUF
                                  : (kMHalves == 2)          ? SMEM_TALL_PAD
                                                             : 4 * SMEM_EPI_T_WARP;
  static constexpr int SMEM_BARRIERS = (2 * kStages + 9) * 8 + 16;
  // +1024: the ring must start on a 1024-byte boundary for the 128-byte swizzle.
  static constexpr int SMEM_TOTAL = kStages * SMEM_STAGE + SMEM_EPI + SMEM_BARRIERS + 1024;
  static constexpr int kAccumCols = BLOCK_N * kMHalves;   // fp32 columns per accumulator set
  static constexpr int kTmemCols = (kCtaGroup == 2 || kNHalves == 2) ? 512
      : (2 * kAccumCols <= 32) ? 32 : (2 * kAccumCols <= 64) ? 64 : (2 * kAccumCols <= 128) ? 128
      : (2 * kAccumCols <= 256) ? 256 : 512;
  static constexpr int kThreads = 64 + 32 * kEpiWarps;   // TMA warp, MMA warp, epilogue warps
  // A configuration that needs less than half of an SM's shared memory is built so that two of
  // its CTAs can share an SM (registers capped accordingly); both then hold a slice of tensor
  // memory at once, which is safe as long as two slices fit.
  static constexpr int kCtasPerSm = (SMEM_TOTAL <= 115712) ? 2 : 1;
  static_assert(kCtasPerSm == 1 || kTmemCols <= 256, "two resident CTAs must both fit in TMEM");
  static_assert(BLOCK_N % 16 == 0 && BLOCK_N >= 16 && BLOCK_N <= 256, "UMMA N");
  static_assert(kNHalves == 1 || (kNHalves == 2 && BLOCK_N == 256 && kEpiMode == kEpiTmaStore),
                "the two-half tile fills tensor memory: 2 x 256 fp32 columns, TMA-store epilogue");
  static_assert(SMEM_Y % 1024 == 0 || kStages == 1 || (SMEM_STAGE % 1024 == 0), "swizzle align");
  static_assert(SMEM_STAGE % 1024 == 0, "every stage must keep 1024-byte alignment");
  static_assert(kEpiMode == kEpiDirect || BLOCK_N % EPI_COLS == 0, "TMA-store boxes are 64 wide");
  static_assert(kCtaGroup == 1 || kTmemCols == 512,
                "pair mode allocates all of tensor memory so both CTAs get column 0");
  static_assert(SMEM_TOTAL <= 232448, "exceeds 227 KB of shared memory per CTA");
  static_assert(kMHalves == 1 || SMEM_STAGE + SMEM_EPI >= 2 * SMEM_X_HALF,
                "the second MMA block of a tall tile reads 256 rows from a slot's start");
  static_assert(kMHalves == 1 || BLOCK_N * kTallRows * 2 <= kStages * SMEM_STAGE,
                "a tall tile stages its whole result in the idle ring");
  static_assert(kMHalves == 1 || (kMHalves == 2 && kNHalves == 1 && kEpiMode == kEpiDirect &&
                                  2 * kAccumCols <= 512),
                "two M-halves: direct-store kernels with both accumulator sets in TMEM");
  // The last tile's store epilogue borrows one 4 KB box buffer per box from the idle ring.
  static_assert(kEpiMode != kEpiTmaStore ||
                    kEpiWarps * 4 * SMEM_EPI_WARP_BUF <= kStages * SMEM_STAGE,
                "the ring must hold every box of a tile");
};

// One unit of work for a CTA (pair).
struct Segment {
  int tile;       // linear tile index
  int kb_begin;   // first k-block
  int kb_count;   // k-blocks in this segment (>= 1)
  int contrib;    // index of this segment among the tile's contributors (0 if whole)
  int n_contrib;  // contributors of this tile (1 if whole)
  int sk_slot;    // index of the tile inside the stream-K region (workspace slot)
};

// Enumerates this CTA's segments.  Every role constructs one and walks the same sequence.
struct SegmentIter {
  int num_k_blocks, real_k_blocks, dyn_ppt, dyn_piece_kb;
  // round-robin part: tiles [0, dp_tiles)
  int next_tile, tile_step, dp_tiles;
  // stream-K part: tiles [sk_first, sk_first + sk_tiles); this CTA's unit range [u0, u1) is cut
  // into head partial, tail partial and whole tiles
  int sk_first, sk_tiles;
  long long u0, u1, head_end, tail_begin, whole, total_units;
  int num_ctas, phase, splits, worker_id;

  __host__ __device__ __forceinline__ SegmentIter(const GemmParams& p, int worker, int num_workers) {
    // With a dynamic tail pool the static ranges only cover the first dyn_static_kb k-blocks of
    // every tile; `num_k_blocks` is the per-tile length of that static unit space.
    dyn_ppt = p.dyn_pieces > 0 ? p.dyn_ppt : 0;
    dyn_piece_kb = p.dyn_piece_kb;
    real_k_blocks = p.num_k_blocks;
    num_k_blocks = dyn_ppt > 0 ? p.dyn_static_kb : p.num_k_blocks;
    next_tile = worker;
    tile_step = num_workers;
    num_ctas = num_workers;
    sk_first = p.stream_k ? p.sk_first_tile : p.num_tiles;
    sk_tiles = p.num_tiles - sk_first;
    dp_tiles = sk_first;
    total_units = static_cast<long long>(sk_tiles) * num_k_blocks;
    phase = sk_tiles > 0 ? 0 : 3;
    splits = p.stream_k ? p.sk_splits : 0;
    worker_id = worker;
    u0 = u1 = head_end = tail_begin = whole = 0;
    // Only launches with cut tiles pay for the 64-bit divisions below: they sit in front of
    // every role's first action (the producer's first copy included).
    if (total_units > 0 && splits == 0) {
      const long long nk = num_k_blocks > 0 ? num_k_blocks : 1;
      u0 = range_start(worker);
      u1 = range_start(worker + 1);
      head_end = u0;
      if (u0 % nk != 0) {
        head_end = (u0 / nk + 1) * nk;
        if (head_end > u1) head_end = u1;
      }
      tail_begin = u1;
      if (u1 % nk != 0 && (u1 / nk) * nk >= head_end) tail_begin = (u1 / nk) * nk;
      whole = head_end;
    }
  }

  __host__ __device__ __forceinline__ long long range_start(int c) const {
    return (total_units * c) / num_ctas;
  }

  // Index of the CTA whose range holds unit `x`.
  __host__ __device__ __forceinline__ int owner_of(long long x) const {
    int c = static_cast<int>((x * num_ctas) / total_units);
    while (c + 1 < num_ctas && range_start(c + 1) <= x) ++c;
    while (c > 0 && range_start(c) > x) --c;
    return c;
  }

  __host__ __device__ __forceinline__ void emit(Segment& s, long long a, long long b) const {
    const int slot = static_cast<int>(a / num_k_blocks);
    const long long tile_u0 = static_cast<long long>(slot) * num_k_blocks;
    s.tile = sk_first + slot;
    s.sk_slot = slot;
    s.kb_begin = static_cast<int>(a - tile_u0);
    s.kb_count = static_cast<int>(b - a);
    if (s.kb_count == num_k_blocks) {
      s.contrib = 0;
      s.n_contrib = 1 + dyn_ppt;
    } else {
      const int first = owner_of(tile_u0);
      const int last = owner_of(tile_u0 + num_k_blocks - 1);
      s.contrib = owner_of(a) - first;
      s.n_contrib = last - first + 1 + dyn_ppt;
    }
  }

  // Segment of dynamic piece `id`: piece j of tile slot id / dyn_ppt, after that tile's static
  // contributors in the summation order.
  __host__ __device__ __forceinline__ void piece(Segment& s, int id) const {
    const int slot = id / dyn_ppt;
    const int j = id - slot * dyn_ppt;
    const long long tile_u0 = static_cast<long long>(slot) * num_k_blocks;
    const int n_static = owner_of(tile_u0 + num_k_blocks - 1) - owner_of(tile_u0) + 1;
    s.tile = sk_first + slot;
    s.sk_slot = slot;
    s.kb_begin = num_k_blocks + j * dyn_piece_kb;
    const int left = real_k_blocks - s.kb_begin;
    s.kb_count = left < dyn_piece_kb ? left : dyn_piece_kb;
    s.contrib = n_static + j;
    s.n_contrib = n_static + dyn_ppt;
  }

  // Order: the stream-K share first (its two partial segments, then its whole tiles), the
  // round-robin tiles last.  A cut tile costs its contributors a round trip through the fp32
  // workspace; doing that early hides it under the main loop of the following segments, and the
  // CTA ends on a plain epilogue.
  __host__ __device__ __forceinline__ bool next(Segment& s) {
    if (phase == 0 && splits > 0) {
      // Uniform cut: all workers holding chunk i of their tiles walk the same k range at the
      // same time, so tiles that share a row or column panel still share it in L2.
      phase = 3;
      const int chunk = worker_id / sk_tiles;
      if (chunk < splits) {
        const int slot = worker_id - chunk * sk_tiles;
        const int kb0 = static_cast<int>(static_cast<long long>(num_k_blocks) * chunk / splits);
        const int kb1 = static_cast<int>(static_cast<long long>(num_k_blocks) * (chunk + 1) / splits);
        s.tile = sk_first + slot;
        s.sk_slot = slot;
        s.kb_begin = kb0;
        s.kb_count = kb1 - kb0;
        s.contrib = splits > 1 ? chunk : 0;
        s.n_contrib = splits;
        return true;
      }
    }
    if (phase == 0) {
      phase = 1;
      if (head_end > u0) {
        emit(s, u0, head_end);
        return true;
      }
    }
    if (phase == 1) {
      phase = 2;
      if (u1 > tail_begin) {
        emit(s, tail_begin, u1);
        return true;
      }
    }
    if (phase == 2) {
      if (whole < tail_begin) {
        emit(s, whole, whole + num_k_blocks);
        whole += num_k_blocks;
        return true;
      }
      phase = 3;
    }
    if (next_tile >= dp_tiles) return false;
    s.tile = next_tile;
    s.sk_slot = 0;
    s.kb_begin = 0;
    s.kb_count = num_k_blocks;
    s.contrib = 0;
    s.n_contrib = 1;
    next_tile += tile_step;
    return true;
  }
};

// Grouped, serpentine raster: consecutive tile ids walk down `group_m` tile rows before moving one
// tile column on, so the tiles in flight at any moment share a few row panels of X and a few
// column panels of Y in L2; the direction across the columns alternates from group to group.  (The reference rasters row-major, neogemmV02.cu:190-191.)
__host__ __device__ __forceinline__ void tile_coords(const GemmParams& p, int tile, int& tm, int& tn) {
  const int group_size = p.group_m * p.num_n_tiles;
  const int group = tile / group_size;
  const int first_m = group * p.group_m;
  const int left = p.num_m_tiles - first_m;
  const int rows = p.group_m < left ? p.group_m : left;
  const int local = tile - group * group_size;
  tm = first_m + local % rows;
  tn = local / rows;
  // Odd groups walk the tile columns backwards: the column panels of Y that the previous group
  // touched last are the first ones the next group asks for, while they are still in L2.
  if (group & 1) tn = p.num_n_tiles - 1 - tn;
}

// Phase timers, the counterpart of the per-CTA load/compute/store cycle records the reference's
// harness reserves a buffer for but never fills (cublass/matmul.cu:99-106,151-165).  Slots per CTA:
//   0 producer: cycles waiting for a free ring slot     1 producer: whole loop
//   2 MMA: cycles waiting for operand bytes             3 MMA: cycles waiting for a drained accumulator
//   4 MMA: whole loop                                   5 epilogue warp 2: waiting for an accumulator
//   6 epilogue warp 2: whole loop                       7 segments processed
//   8 CTA start   9 MMA loop start   10 MMA loop end   11 epilogue loop end   12 CTA end
//   (8..12 are %globaltimer nanoseconds, so that CTAs can be laid on one time axis)
struct PhaseTimer {
  long long* slot;
  long long t0, sum;
  __device__ __forceinline__ PhaseTimer(const GemmParams& p) {
    slot = p.timers ? p.timers + static_cast<long long>(blockIdx.x) * 16 : nullptr;
    t0 = 0;
    sum = 0;
  }
  __device__ __forceinline__ void begin() { if (slot) t0 = clock64(); }
  // Accumulates in a register; flush() writes the sum once, after the role's loop.
  __device__ __forceinline__ void end() { if (slot) sum += clock64() - t0; }
  __device__ __forceinline__ void flush(int i) { if (slot) slot[i] += sum; }
  __device__ __forceinline__ void stamp(int i) {
    if (slot) slot[i] = static_cast<long long>(ptx::globaltimer_ns());
  }
};

__device__ __forceinline__ void report_error(const GemmParams& p, volatile int* abort_flag,
                                             int code, int seg, int aux) {
  *abort_flag = 1;
  if (p.status != nullptr && atomicCAS(p.status, 0, code) == 0) {
    p.status[1] = static_cast<int>(blockIdx.x);
    p.status[2] = seg;
    p.status[3] = aux;
    __threadfence_system();
  }
}

// Wave pacing.  SM clocks differ by a few per cent between GPCs, so with a static round-robin
// schedule the workers drift apart over a long launch (55 waves at 65536 x 8192 x 8192: the
// fastest are whole tiles ahead by the end).  Tiles of one wave share their operand panels through
// L2 only while they walk K roughly together; once the drift exceeds what L2 holds, every worker
// fetches its panels from DRAM on its own (measured there: 9.7 GB read against 6.2 GB by cuBLAS and
// 6.9 GB for workers in step), and on a power-capped GPU the extra traffic costs clock.
// So the producer of every worker (the leader CTA of a pair) reports its arrival at the start of
// each wave after the first and waits until all workers with a tile in that wave have arrived.
// The launch ends with its slowest worker either way; the fast ones idle between waves instead of
// at the end.  The wait is soft: it gives up after pace_timeout_ns and nothing depends on it.
// The counter returns to zero with the launch's last arrival.
__device__ __forceinline__ void pace_wave(const GemmParams& p, int wave, int num_workers,
                                          uint32_t lane) {
  if (lane == 0) {
    const int total = p.num_tiles - num_workers;                    // arrivals of the whole launch
    const int in_wave = min(num_workers, p.num_tiles - wave * num_workers);
    const int need = (wave - 1) * num_workers + in_wave;            // all of this wave have arrived
    const int mine = atomicAdd(p.pace_counter, 1) + 1;
    if (mine == total) {
      *reinterpret_cast<volatile int*>(p.pace_counter) = 0;          // nobody arrives after this
    } else if (mine < need) {
      const uint64_t t0 = ptx::globaltimer_ns();
      for (;;) {
        const int seen = *reinterpret_cast<volatile int*>(p.pace_counter);
        // seen < mine: the counter was reset, i.e. the launch's last arrival has happened
        if (seen >= need || seen < mine) break;
        if (ptx::globaltimer_ns() - t0 > static_cast<uint64_t>(p.pace_timeout_ns)) break;
        __nanosleep(100);
      }
    }
  }
  __syncwarp();
}

// Where a role gets its segments from: first the static sequence every role derives on its own
// (SegmentIter), then - if the launch has a dynamic tail pool - pieces claimed at run time.  The
// TMA warp claims (atomicAdd on a global counter) and publishes each claim to the MMA warp and
// the four epilogue warps through a two-slot queue in shared memory guarded by mbarriers; -1
// ends the stream.  Waits are bounded like every other wait in the kernel.
struct WorkSource {
  SegmentIter it;
  uint32_t sched_full, sched_empty;   // [2] each
  volatile int* ids;                  // [2]
  const volatile int* abort_flag;
  uint32_t q, qphase;
  bool is_claimer, done, failed;
  int dyn_pieces, num_workers;
  int* dyn_counter;

  __device__ __forceinline__ WorkSource(const GemmParams& p, int worker, int workers, bool claimer,
                                        uint32_t full_bar, uint32_t empty_bar, volatile int* ids_,
                                        const volatile int* abort)
      : it(p, worker, workers), sched_full(full_bar), sched_empty(empty_bar), ids(ids_),
        abort_flag(abort), q(0), qphase(0), is_claimer(claimer), done(p.dyn_pieces == 0),
        failed(false), dyn_pieces(p.dyn_pieces), num_workers(workers), dyn_counter(p.dyn_counter) {}

  // Warp-collective: all 32 lanes call it together and get the same answer.
  __device__ __forceinline__ bool next(Segment& s, uint32_t lane) {
    if (it.next(s)) return true;
    if (done) return false;
    int id = -1;
    if (is_claimer) {
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(sched_empty + 8 * q, qphase ^ 1, abort_flag))) {
        failed = done = true;
        return false;
      }
      if (lane == 0) {
        const int got = atomicAdd(dyn_counter, 1);
        // Every CTA claims until it draws an id past the end, exactly once: the launch makes
        // dyn_pieces + num_workers claims in total, and the last one resets the counter.
        if (got == dyn_pieces + num_workers - 1) *dyn_counter = 0;
        id = got < dyn_pieces ? got : -1;
        ids[q] = id;
        ptx::mbar_arrive(sched_full + 8 * q);   // release: publishes ids[q]
      }
      id = __shfl_sync(0xffffffffu, id, 0);
    } else {
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(sched_full + 8 * q, qphase, abort_flag))) {
        failed = done = true;
        return false;
      }
      id = ids[q];
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(sched_empty + 8 * q);
    }
    q ^= 1;
    if (q == 0) qphase ^= 1;
    if (id < 0) {
      done = true;
      return false;
    }
    it.piece(s, id);
    return true;
  }
};

// Fused epilogue on kN consecutive columns [col, col + kN) of one row of D held in r[] (fp32
// bit patterns), in place.  Reads of C_in and bias are bounds-checked against Md / Nd.
// kF32: the instantiation may be asked for an fp32 result (beta term read from c_in32); kernels
// that never are (two-half tiles) compile the branch out, it would only cost them registers.
template <int kN, bool kF32 = true>
__device__ __forceinline__ void fused_epilogue(uint32_t (&r)[kN], const GemmParams& p, int row,
                                               int col) {
  const bool row_ok = row < p.Md;
  float row_bias = 0.f;
  if (p.bias != nullptr && p.bias_on_rows && row_ok) row_bias = __bfloat162float(p.bias[row]);
  const __nv_bfloat16* cin = nullptr;
  const float* cin32 = nullptr;
  if (p.beta != 0.f && row_ok) {
    if (kF32 && p.c_in32 != nullptr) cin32 = p.c_in32 + static_cast<long long>(row) * p.out_stride_r;
    else cin = p.c_in + static_cast<long long>(row) * p.out_stride_r;
  }
#pragma unroll
  for (int j = 0; j < kN; ++j) {
    float v = p.alpha * __uint_as_float(r[j]);
    const bool ok = row_ok && (col + j) < p.Nd;
    if (cin != nullptr && ok)
      v += p.beta * __bfloat162float(cin[static_cast<long long>(col + j) * p.out_stride_c]);
    if (kF32 && cin32 != nullptr && ok)
      v += p.beta * cin32[static_cast<long long>(col + j) * p.out_stride_c];
    if (p.bias != nullptr && ok)
      v += p.bias_on_rows ? row_bias : __bfloat162float(p.bias[col + j]);
    if (p.activation == 1) {
      v = fmaxf(v, 0.f);
    } else if (p.activation == 2) {
      const float u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
      v = 0.5f * v * (1.f + tanhf(u));
    }
    r[j] = __float_as_uint(v);
  }
}

// Stream-K fix-up of kN accumulator columns held by one thread (one row): replaces r[] by the
// sum of all contributors' partials in contributor order, taking this contributor's own value
// from r[] itself, so the result does not depend on which contributor arrived last.  `col_base`
// points at this row's entry of the first of the kN columns in contributor 0's slot; consecutive
// columns are `col_stride` floats apart and consecutive contributors `slot_stride`.
template <int kN, int kGroup = ((kN <= 16) ? 4 : 1)>
__device__ __forceinline__ void sum_partials(uint32_t (&r)[kN], const float* col_base,
                                             size_t col_stride, size_t slot_stride, int contrib,
                                             int n_contrib) {
  // Up to kGroup contributors' loads are issued before any is consumed (kGroup * kN independent
  // loads in flight per thread, each a 128-byte line per warp), then added in contributor order.
  float sum[kN];
#pragma unroll 1
  for (int q0 = 0; q0 < n_contrib; q0 += kGroup) {
    float t[kGroup][kN];
#pragma unroll
    for (int g = 0; g < kGroup; ++g) {
      const int q = q0 + g;
      if (q < n_contrib && q != contrib) {
        const float* src = col_base + static_cast<size_t>(q) * slot_stride;
#pragma unroll
        for (int j = 0; j < kN; ++j) t[g][j] = __ldcg(src + static_cast<size_t>(j) * col_stride);
      }
    }
#pragma unroll
    for (int g = 0; g < kGroup; ++g) {
      const int q = q0 + g;
      if (q < n_contrib) {
#pragma unroll
        for (int j = 0; j < kN; ++j) {
          const float v = (q == contrib) ? __uint_as_float(r[j]) : t[g][j];
          sum[j] = (q == 0) ? v : sum[j] + v;
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < kN; ++j) r[j] = __float_as_uint(sum[j]);
}

template <class Cfg>
__global__ void __launch_bounds__(Cfg::kThreads, Cfg::kCtasPerSm)
gemm_bf16_nt_kernel(const __grid_constant__ CUtensorMap tmap_x,
                    const __grid_constant__ CUtensorMap tmap_y,
                    const __grid_constant__ CUtensorMap tmap_d,
                    const GemmParams p) {
  using namespace ptx;
  constexpr int kCtaGroup = Cfg::kCtaGroup;
  constexpr int BLOCK_N = Cfg::BLOCK_N;
  constexpr int kStages = Cfg::kStages;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const uint32_t ring = smem_base;
  const uint32_t epi_base = ring + kStages * Cfg::SMEM_STAGE;
  const uint32_t bar_base = epi_base + Cfg::SMEM_EPI;
  const uint32_t full_bar = bar_base;                       // [kStages]
  const uint32_t empty_bar = full_bar + 8 * kStages;        // [kStages]
  const uint32_t tmem_full_bar = empty_bar + 8 * kStages;   // [2]
  const uint32_t tmem_empty_bar = tmem_full_bar + 16;       // [2]
  const uint32_t sched_full_bar = tmem_empty_bar + 16;      // [2] dynamic-claim queue
  const uint32_t sched_empty_bar = sched_full_bar + 16;     // [2]
  const uint32_t epi_sync_bar = sched_empty_bar + 16;       // [1] tall tiles: result staged
  const uint32_t tmem_slot = epi_sync_bar + 8;              // u32
  uint8_t* tail_gen = smem_gen + (tmem_slot - smem_base);
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(tail_gen);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail_gen + 4);
  volatile int* sched_ids = reinterpret_cast<volatile int*>(tail_gen + 8);   // [2]

  const int warp = threadIdx.x >> 5;
  const uint32_t lane = lane_id();
  const uint32_t cta_rank = (kCtaGroup == 2) ? cluster_ctarank() : 0u;
  const bool is_leader = (cta_rank == 0);
  const int worker = static_cast<int>(blockIdx.x) / kCtaGroup;
  const int num_workers = static_cast<int>(gridDim.x) / kCtaGroup;

  // ---------------------------------------------------------------- set-up
  // Everything down to griddep_wait() works on shared memory, tensor memory and kernel
  // parameters only, so it may run while the previous kernel of the stream is still finishing.
  if (threadIdx.x == 0) {
    griddep_launch_dependents();
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar + 8 * s, 1);   // one arrive.expect_tx per phase (leader's producer)
      mbar_init(empty_bar + 8 * s, 1);  // one tcgen05.commit per phase
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tmem_full_bar + 8 * a, 1);               // one tcgen05.commit per tile
      // one arrive per epilogue warp that reads the accumulator (all of them for two-half tiles)
      mbar_init(tmem_empty_bar + 8 * a, Cfg::kEpiWarps * kCtaGroup);
      mbar_init(sched_full_bar + 8 * a, 1);                   // the claiming lane
      mbar_init(sched_empty_bar + 8 * a, 1 + Cfg::kEpiWarps); // MMA warp + epilogue warps
    }
    mbar_init(epi_sync_bar, 4);   // the four epilogue warps of a tall tile
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tmap_x);
    prefetch_tensormap(&tmap_y);
    if (Cfg::kEpiMode == kEpiTmaStore || (Cfg::kMHalves == 2 && (p.l2_hints & 96)))
      prefetch_tensormap(&tmap_d);
  }
  if (warp == 1) {
    tmem_alloc<1>(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish<1>();
  }
  tcgen05_fence_before();
  if (kCtaGroup == 2) cluster_sync_all(); else __syncthreads();
  tcgen05_fence_after();
  // From here on global memory is read and written: wait for the previous kernel of the stream
  // (a no-op for launches without the programmatic-serialization attribute).
  griddep_wait();
  if (threadIdx.x == 0) PhaseTimer(p).stamp(8);
  const uint32_t tmem_base = *tmem_slot_gen;
  if (kCtaGroup == 2 && tmem_base != 0 && threadIdx.x == 0) {
    // The pair's MMA addresses both CTAs' tensor memory with the leader's address.
    report_error(p, abort_flag, kDevTmemAddress, 0, static_cast<int>(tmem_base));
  }
  if (kCtaGroup == 2) __syncthreads();

  // ---------------------------------------------------------------- roles
  if (warp == 0) {
    // ======================= TMA producer =======================
    // The whole warp walks the loop so that every loop-carried value stays warp-uniform; one
    // elected lane issues the copies.
    if (*abort_flag == 0) {
      WorkSource it(p, worker, num_workers, true, sched_full_bar, sched_empty_bar, sched_ids,
                    abort_flag);
      Segment seg;
      uint32_t stage = 0, phase = 0;
      int seg_idx = 0;
      const uint32_t leader_full = (kCtaGroup == 2) ? mapa_u32(full_bar, 0) : full_bar;
      // X is the operand the raster keeps across consecutive waves (a group of tile rows); Y
      // streams past it.
      const bool hint_x = (p.l2_hints & 9) != 0, hint_y = (p.l2_hints & 18) != 0;
      const uint64_t pol_x = (p.l2_hints & 8) ? l2_policy_evict_first() : l2_policy_evict_last();
      const uint64_t pol_y = (p.l2_hints & 16) ? l2_policy_evict_last() : l2_policy_evict_first();
      bool ok = true;
      GemmParams timer_params = p;
      if (lane != 0) timer_params.timers = nullptr;
      PhaseTimer wait_timer(timer_params), loop_timer(timer_params);
      loop_timer.begin();
      int first_fill = 0;   // k-blocks issued so far, counted up to the ring's depth
      while (ok && it.next(seg, lane)) {
        if (p.pace_counter != nullptr && is_leader && seg_idx >= 1)
          pace_wave(p, seg_idx, num_workers, lane);
        int tm, tn;
        tile_coords(p, seg.tile, tm, tn);
        // Tall tiles: every CTA (of a pair, too) owns tile_rows consecutive rows of X.
        const int row_x = (Cfg::kMHalves == 2)
            ? (tm * kCtaGroup + static_cast<int>(cta_rank)) * p.tile_rows
            : tm * Cfg::TILE_M + static_cast<int>(cta_rank) * Cfg::BLOCK_M;
        // Bytes one stage receives: the X box of a tall tile is tile_rows high.
        const uint32_t stage_bytes = (Cfg::kMHalves == 2)
            ? static_cast<uint32_t>(p.tile_rows) * (Cfg::BLOCK_K * 2) + Cfg::SMEM_Y
            : static_cast<uint32_t>(Cfg::SMEM_STAGE);
        const int row_y = tn * Cfg::TILE_N + static_cast<int>(cta_rank) * Cfg::LOAD_N;
        const int kb_end = seg.kb_begin + seg.kb_count;
        // Only the producer knows the direction: the MMA warp consumes ring slots in order and
        // the sum of a tile's k-blocks does not care which came first (the order is fixed per
        // tile, so results stay reproducible).
        const bool reverse_k = p.k_alternate != 0 && (seg_idx & 1) != 0 && seg.n_contrib == 1;
        for (int kb = seg.kb_begin; kb < kb_end; ++kb) {
          // The first pass over the ring finds every slot free: no MMA has read it yet, so
          // there is nothing to wait for (a wait that passes at once still costs ~150 cycles,
          // which a launch of a few k-blocks per CTA feels: it is the rate its loads go out at).
          bool got = true;
          if (Cfg::kNHalves == 2 || first_fill >= kStages) {
            wait_timer.begin();
            got = __all_sync(0xffffffffu,
                             mbar_wait(empty_bar + 8 * stage, phase ^ 1, abort_flag,
                                       static_cast<uint32_t>(p.main_wait_hint_ns)));
            wait_timer.end();
          } else {
            ++first_fill;
          }
          if (!got) {
            if (lane == 0)
              report_error(p, abort_flag, kDevTimeoutProducer, seg_idx, static_cast<int>(stage));
            ok = false;
            break;
          }
          const uint32_t sx = ring + stage * Cfg::SMEM_STAGE;
          const uint32_t sy = sx + Cfg::SMEM_X;
          if (elect_one()) {
            const int c0 = (reverse_k ? (seg.kb_begin + kb_end - 1 - kb) : kb) * Cfg::BLOCK_K;
            if (kCtaGroup == 1) {
              mbar_arrive_expect_tx(full_bar + 8 * stage, stage_bytes);
              if (hint_x) tma_load_2d_hint(sx, &tmap_x, full_bar + 8 * stage, c0, row_x, pol_x);
              else tma_load_2d(sx, &tmap_x, full_bar + 8 * stage, c0, row_x);
#pragma unroll
              for (int h = 0; h < Cfg::kNHalves; ++h) {
                const uint32_t dst = sy + h * Cfg::SMEM_Y_HALF;
                const int ry = row_y + h * BLOCK_N;
                if (hint_y) tma_load_2d_hint(dst, &tmap_y, full_bar + 8 * stage, c0, ry, pol_y);
                else tma_load_2d(dst, &tmap_y, full_bar + 8 * stage, c0, ry);
              }
            } else {
              if (is_leader) mbar_arrive_expect_tx(full_bar + 8 * stage, 2 * stage_bytes);
              if (hint_x) tma_load_2d_pair_hint(sx, &tmap_x, leader_full + 8 * stage, c0, row_x, pol_x);
              else tma_load_2d_pair(sx, &tmap_x, leader_full + 8 * stage, c0, row_x);
#pragma unroll
              for (int h = 0; h < Cfg::kNHalves; ++h) {
                const uint32_t dst = sy + h * Cfg::SMEM_Y_HALF;
                const int ry = row_y + h * BLOCK_N;
                if (hint_y) tma_load_2d_pair_hint(dst, &tmap_y, leader_full + 8 * stage, c0, ry, pol_y);
                else tma_load_2d_pair(dst, &tmap_y, leader_full + 8 * stage, c0, ry);
              }
            }
          }
          __syncwarp();
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        ++seg_idx;
      }
      if (it.failed && lane == 0) report_error(p, abort_flag, kDevTimeoutScheduler, seg_idx, 0);
      loop_timer.end();
      loop_timer.flush(1);
      wait_timer.flush(0);
    }
    __syncwarp();
  } else if (warp == 1) {
    // ======================= UMMA issuer (leader CTA only) =======================
    // Warp-uniform loop, one elected lane issues tcgen05.mma / tcgen05.commit.
    if (is_leader && *abort_flag == 0) {
      WorkSource it(p, worker, num_workers, false, sched_full_bar, sched_empty_bar, sched_ids,
                    abort_flag);
      Segment seg;
      uint32_t stage = 0, phase = 0;
      int seg_idx = 0;
      constexpr uint32_t idesc = make_idesc_bf16(Cfg::UMMA_M, BLOCK_N);
      const uint32_t idesc_flip0 = make_idesc_bf16(128, 256);
      const uint32_t idesc_flip1 =
          make_idesc_bf16(128, static_cast<uint32_t>(2 * max(p.tile_rows - 128, 8)));
      bool ok = true;
      GemmParams timer_params = p;
      if (lane != 0) timer_params.timers = nullptr;
      PhaseTimer wait_timer(timer_params), tmem_timer(timer_params), loop_timer(timer_params);
      loop_timer.stamp(9);
      loop_timer.begin();
      while (ok && it.next(seg, lane)) {
        // One-half tiles alternate between two accumulators (two tiles in flight); a two-half
        // tile owns both, and each half is waited for just before its first MMA.
        const uint32_t acc = (Cfg::kNHalves == 1) ? (seg_idx & 1) : 0;
        const uint32_t acc_phase = (Cfg::kNHalves == 1) ? ((seg_idx >> 1) & 1) : (seg_idx & 1);
        if (Cfg::kNHalves == 1) {
          tmem_timer.begin();
          const bool drained = __all_sync(
              0xffffffffu,
              mbar_wait<kCtaGroup == 2>(tmem_empty_bar + 8 * acc, acc_phase ^ 1, abort_flag));
          tmem_timer.end();
          if (!drained) {
            if (lane == 0)
              report_error(p, abort_flag, kDevTimeoutMmaTmem, seg_idx, static_cast<int>(acc));
            break;
          }
          tcgen05_fence_after();
        }
        const uint32_t tmem_d = tmem_base + acc * Cfg::kAccumCols;
        // Encoded distance between the two Y halves of a stage (16-byte units).
        constexpr uint64_t kHalfStep = Cfg::SMEM_Y_HALF >> 4;
        int kb_first = 0;
        if (Cfg::kNHalves == 2) {
          // Prologue of a two-half tile.  Half 0 comes back from the epilogue first, half 1 a
          // little later, so the first k-blocks (as many as the ring holds minus one) are issued
          // for half 0 alone, then, once half 1 is back, for half 1 - which also releases their
          // ring slots.  The tensor pipe restarts as soon as half 0 is drained.
          const int pro = min(min(kStages - 1, max(p.wide_prologue, 1)), seg.kb_count);
#pragma unroll 1
          for (int h = 0; h < 2 && ok; ++h) {
            tmem_timer.begin();
            const bool drained = __all_sync(
                0xffffffffu,
                mbar_wait<kCtaGroup == 2, true>(tmem_empty_bar + 8 * h, acc_phase ^ 1, abort_flag));
            tmem_timer.end();
            if (!drained) {
              if (lane == 0) report_error(p, abort_flag, kDevTimeoutMmaTmem, seg_idx, h);
              ok = false;
              break;
            }
            tcgen05_fence_after();
            uint32_t st = stage, ph = phase;
#pragma unroll 1
            for (int j = 0; j < pro; ++j) {
              if (h == 0) {
                wait_timer.begin();
                const bool got = __all_sync(
                    0xffffffffu, mbar_wait(full_bar + 8 * st, ph, abort_flag,
                                           static_cast<uint32_t>(p.main_wait_hint_ns)));
                wait_timer.end();
                if (!got) {
                  if (lane == 0)
                    report_error(p, abort_flag, kDevTimeoutMmaFull, seg_idx, static_cast<int>(st));
                  ok = false;
                  break;
                }
                tcgen05_fence_after();
              }
              const uint32_t sx = ring + st * Cfg::SMEM_STAGE;
              const uint64_t desc_x = make_smem_desc_sw128(sx);
              const uint64_t desc_y = make_smem_desc_sw128(sx + Cfg::SMEM_X) + h * kHalfStep;
              if (elect_one()) {
#pragma unroll
                for (int k = 0; k < Cfg::BLOCK_K / Cfg::UMMA_K; ++k)
                  umma_bf16<kCtaGroup>(tmem_d + h * Cfg::kAccumCols, desc_x + 2 * k, desc_y + 2 * k,
                                       idesc, (j > 0 || k > 0) ? 1u : 0u);
                if (h == 1) {
                  if (kCtaGroup == 2) umma_commit_both_ctas(empty_bar + 8 * st);
                  else umma_commit<1>(empty_bar + 8 * st);
                }
              }
              __syncwarp();
              if (++st == kStages) { st = 0; ph ^= 1; }
            }
            if (h == 1 && ok) { stage = st; phase = ph; }
          }
          if (!ok) break;
          kb_first = pro;
        }
        // Two-half tiles: early notice to the epilogue warps of both CTAs a few k-blocks before the
        // tile's last MMA is issued (they wake from a suspended wait, which can take microseconds,
        // and then poll the accumulator barrier).
        const int notice_kb = max(kb_first, seg.kb_count - 3);
        bool noticed = false;
        for (int kb = kb_first; kb < seg.kb_count; ++kb) {
          if (Cfg::kNHalves == 2 && kb == notice_kb) {
            if (elect_one()) {
              mbar_arrive(tmem_full_bar + 8);
              if (kCtaGroup == 2) mbar_arrive_cluster(mapa_u32(tmem_full_bar + 8, 1));
            }
            noticed = true;
          }
          wait_timer.begin();
          const bool got = __all_sync(0xffffffffu,
                                      mbar_wait(full_bar + 8 * stage, phase, abort_flag,
                                                static_cast<uint32_t>(p.main_wait_hint_ns)));
          wait_timer.end();
          if (!got) {
            if (lane == 0)
              report_error(p, abort_flag, kDevTimeoutMmaFull, seg_idx, static_cast<int>(stage));
            ok = false;
            break;
          }
          tcgen05_fence_after();
          const uint32_t sx = ring + stage * Cfg::SMEM_STAGE;
          const uint64_t desc_x = make_smem_desc_sw128(sx);
          const uint64_t desc_y = make_smem_desc_sw128(sx + Cfg::SMEM_X);
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < Cfg::BLOCK_K / Cfg::UMMA_K; ++k) {
              // +32 bytes (two 16-byte units) per 16-element K step inside the swizzle row.
              if constexpr (Cfg::kFlippable) {
                if (p.l2_hints & 64) {
                  // Roles exchanged (see kFlippable): Y's 2 x 64 rows are the M side, X's rows
                  // the N side - 2 x 128 of them in the first instruction, the 2 x (tile_rows -
                  // 128) below them in the second, whose columns follow in tensor memory.
                  umma_bf16<kCtaGroup>(tmem_d, desc_y + 2 * k, desc_x + 2 * k, idesc_flip0,
                                       (kb > 0 || k > 0) ? 1u : 0u);
                  umma_bf16<kCtaGroup>(tmem_d + 128, desc_y + 2 * k,
                                       desc_x + (Cfg::SMEM_X_HALF >> 4) + 2 * k, idesc_flip1,
                                       (kb > 0 || k > 0) ? 1u : 0u);
                  continue;
                }
              }
              if constexpr (Cfg::kMHalves == 2) {
                // Two blocks of X rows, one Y: the second block sits SMEM_X_HALF further on.
#pragma unroll
                for (int mh = 0; mh < 2; ++mh)
                  umma_bf16<kCtaGroup>(tmem_d + mh * BLOCK_N,
                                       desc_x + mh * (Cfg::SMEM_X_HALF >> 4) + 2 * k, desc_y + 2 * k,
                                       idesc, (kb > 0 || k > 0) ? 1u : 0u);
              } else {
#pragma unroll
                for (int h = 0; h < Cfg::kNHalves; ++h)
                  umma_bf16<kCtaGroup>(tmem_d + h * Cfg::kAccumCols, desc_x + 2 * k,
                                       desc_y + h * kHalfStep + 2 * k, idesc,
                                       (kb > 0 || k > 0) ? 1u : 0u);
              }
            }
            if (kCtaGroup == 2) umma_commit_both_ctas(empty_bar + 8 * stage);
            else umma_commit<1>(empty_bar + 8 * stage);
          }
          __syncwarp();
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        if (elect_one()) {
          if (Cfg::kNHalves == 2 && !noticed) {   // short tiles: the loop above did not run
            mbar_arrive(tmem_full_bar + 8);
            if (kCtaGroup == 2) mbar_arrive_cluster(mapa_u32(tmem_full_bar + 8, 1));
          }
          if (kCtaGroup == 2) umma_commit_both_ctas(tmem_full_bar + 8 * acc);
          else umma_commit<1>(tmem_full_bar + 8 * acc);
        }
        __syncwarp();
        ++seg_idx;
      }
      if (it.failed && lane == 0) report_error(p, abort_flag, kDevTimeoutScheduler, seg_idx, 1);
      loop_timer.end();
      loop_timer.stamp(10);
      loop_timer.flush(4);
      wait_timer.flush(2);
      tmem_timer.flush(3);
      if (loop_timer.slot) loop_timer.slot[7] += seg_idx;
    }
    __syncwarp();
  } else {
    // ======================= epilogue (warps 2..5) =======================
    const uint32_t quad = warp & 3;               // TMEM lane quadrant this warp may read
    const int warp_set = (warp - 2) >> 2;         // two-half tiles: which 128 columns of each half
    const int row_in_cta = quad * 32 + lane;      // accumulator row owned by this thread
    const uint32_t leader_tmem_empty = (kCtaGroup == 2) ? mapa_u32(tmem_empty_bar, 0) : 0u;
    WorkSource it(p, worker, num_workers, false, sched_full_bar, sched_empty_bar, sched_ids,
                  abort_flag);
    Segment seg;
    int seg_idx = 0;
    uint32_t store_count = 0;
    const uint64_t pol_d = l2_policy_evict_first();
    bool ok = (*abort_flag == 0);
    GemmParams timer_params = p;
    if (warp != 2 || lane != 0) timer_params.timers = nullptr;
    PhaseTimer wait_timer(timer_params), loop_timer(timer_params);
    loop_timer.begin();
    while (ok && it.next(seg, lane)) {
      if (Cfg::kMHalves == 2 && seg_idx > 0) {
        // A tall tile is its CTA's only tile (the launcher sizes the grid that way): its result
        // is staged in the operand ring, which a second tile's loads would be filling.
        if (lane == 0) report_error(p, abort_flag, kDevBounds, seg_idx, 9);
        break;
      }
      const uint32_t acc = (Cfg::kNHalves == 1) ? (seg_idx & 1) : 0;
      const uint32_t acc_phase = (Cfg::kNHalves == 1) ? ((seg_idx >> 1) & 1) : (seg_idx & 1);
      // Is this the CTA's last segment?  Then, once its accumulator is complete, nothing reads
      // or fills the operand ring any more (every copy issued has been consumed by an MMA that
      // has finished), and the store epilogue may use it as staging: every box of the tile gets
      // a buffer of its own and the TMA stores go out back to back instead of waiting, box by
      // box, for the one or two regular buffers to be read out (~1 us each) - that wait is
      // otherwise the exposed tail of every launch.
      bool ring_is_free = false;
      if (Cfg::kEpiMode == kEpiTmaStore && p.dyn_pieces == 0) {
        SegmentIter peek = it.it;
        Segment unused;
        ring_is_free = !peek.next(unused);
      }
      // Everything that does not need the accumulator is worked out before the wait: with a
      // two-half tile the tensor pipe idles from the moment the barrier fires until this warp has
      // read its share, and the index arithmetic alone was ~1500 cycles of that.
      int tm, tn;
      tile_coords(p, seg.tile, tm, tn);
      const int row0_tile = (Cfg::kMHalves == 2)
          ? (tm * kCtaGroup + static_cast<int>(cta_rank)) * p.tile_rows
          : tm * Cfg::TILE_M + static_cast<int>(cta_rank) * Cfg::BLOCK_M;
      // Rows of D this tile owns end here (tall tiles: the second block is only partly the
      // tile's; everything else: the matrix edge).
      const int row_limit = (Cfg::kMHalves == 2) ? min(p.Md, row0_tile + p.tile_rows) : p.Md;
      const int col0 = tn * Cfg::TILE_N;
      const uint32_t taddr_tile = tmem_base + ((quad * 32u) << 16) + acc * Cfg::kAccumCols;
      const int row0 = row0_tile;            // (the direct-store walk shadows these per M-half)
      const uint32_t taddr = taddr_tile;
      // Pin the values in registers here; otherwise the compiler sinks the arithmetic to its first
      // use, which is behind the wait.
      asm volatile("" ::"r"(row0_tile), "r"(col0), "r"(taddr_tile));
      wait_timer.begin();
      // One lane polls; the other 31 sleep at the shuffle instead of hammering the barrier.
      int got_i = 0;
      // Two-half tiles sleep on the early notice (barrier slot 1, raised when the tile's last MMA
      // has been issued) and then poll the real barrier from inside the read-out loop below.
      // The CTA's last accumulator is awaited with non-blocking tests: nothing hides a late
      // wake-up from a suspended wait there (it can be microseconds), it is the launch's tail.
      if (lane == 0) {
        const uint32_t bar = tmem_full_bar + 8 * (Cfg::kNHalves == 2 ? 1u : acc);
        got_i = (ring_is_free && Cfg::kNHalves == 1)
            ? (mbar_wait<false, true>(bar, acc_phase, abort_flag) ? 1 : 0)
            : (mbar_wait(bar, acc_phase, abort_flag,
                         static_cast<uint32_t>(p.epi_wait_hint_ns)) ? 1 : 0);
      }
      const bool got = __shfl_sync(0xffffffffu, got_i, 0) != 0;
      wait_timer.end();
      if (!got) {
        if (lane == 0) report_error(p, abort_flag, kDevTimeoutEpilogue, seg_idx, static_cast<int>(acc));
        break;
      }
      tcgen05_fence_after();

      // ---- stream-K: publish this segment's partial; the last arriver finishes the rows ----
      bool finish = true;
      const float* tile_partials = nullptr;
      if constexpr (Cfg::kNHalves == 1 && Cfg::kMHalves == 1) {
        if (seg.n_contrib > 1) {
          // Slot layout [contributor][column][row] so that a warp's 32 rows of one column are
          // one 128-byte line.  Counters are per (tile, CTA of the pair, lane quadrant): the
          // four epilogue warps never have to synchronise with each other.
          tile_partials = p.partials + static_cast<size_t>(seg.sk_slot) * p.max_contrib *
                                           (static_cast<size_t>(BLOCK_N) * Cfg::TILE_M);
          float* mine = const_cast<float*>(tile_partials) +
                        static_cast<size_t>(seg.contrib) * BLOCK_N * Cfg::TILE_M +
                        cta_rank * Cfg::BLOCK_M + row_in_cta;
          const long long slot_end = (static_cast<long long>(seg.sk_slot) * p.max_contrib +
                                      seg.contrib + 1) * (static_cast<long long>(BLOCK_N) * Cfg::TILE_M);
          const long long counter_idx =
              (static_cast<long long>(seg.sk_slot) * kCtaGroup + cta_rank) * 4 + quad;
          const bool in_bounds = seg.contrib >= 0 && seg.contrib < p.max_contrib &&
                                 seg.n_contrib <= p.max_contrib && slot_end <= p.partials_elems &&
                                 counter_idx < p.counters_len;
          if (!__all_sync(0xffffffffu, in_bounds)) {
            if (lane == 0) report_error(p, abort_flag, kDevBounds, seg_idx, in_bounds ? 2 : 1);
            break;
          }
#pragma unroll 1
          for (int c = 0; c < BLOCK_N; c += 16) {
            uint32_t r[16];
            __syncwarp();
            tmem_ld_32x32b_x16(taddr + c, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j)
              __stcg(mine + static_cast<size_t>(c + j) * Cfg::TILE_M, __uint_as_float(r[j]));
          }
          // Release: the warp's stores are ordered before lane 0's fence by the warp barrier, and
          // the fence orders them before the counter increment for every other CTA (cumulativity),
          // so one lane fences instead of thirty-two.  Acquire on the way back, same shape.
          __syncwarp();
          if (p.sk_two_pass) {
            finish = false;   // the reduction kernel behind this launch completes the tile
          } else {
            int* counter = p.tile_counters + counter_idx;
            int prev = 0;
            if (lane == 0) {
              __threadfence();
              prev = atomicAdd(counter, 1);
              if (prev == seg.n_contrib - 1) {
                __threadfence();
                *counter = 0;  // ready for the next launch that uses this workspace
              }
            }
            prev = __shfl_sync(0xffffffffu, prev, 0);
            finish = (prev == seg.n_contrib - 1);
          }
        }
      }

      bool transposed = false;
      bool released = false;
      if (!finish) {
        // nothing to store: another contributor completes these rows
      } else
      if constexpr (Cfg::kEpiMode == kEpiTmaStore && Cfg::kNHalves == 2) {
        // Two-half tile: all 512 TMEM columns belong to this tile, so the next tile's MMAs wait
        // for this read-out.  Keep it free of anything slow: this warp's share (32 rows x 128
        // columns of each half) is pulled into registers - half 0, hand it back, pack to bf16,
        // half 1, hand it back, pack - and only then goes through the staging buffer and the TMA
        // stores, whose shared-memory read-out takes about a microsecond per box.
        const uint32_t buf = epi_base + (warp - 2) * Cfg::SMEM_EPI_WARP_BUF;
        const int my_row0 = row0 + quad * 32;
        uint32_t packed[2][64];
        {
          // Half 0 is what the next tile's first MMA waits for.  Its four loads (128 raw
          // registers, free at this point) run in a loop that starts at the early notice and
          // tests the accumulator barrier once per turn: turns before the barrier fires read
          // unfinished sums and are thrown away, but they keep this code and its registers hot,
          // so that the turn which sees the barrier hands the half back ~300 cycles later.  A
          // cold start (wake-up, instruction fetch, spills) cost 2000-3500 cycles per tile.
          const uint32_t t_half = taddr + warp_set * (BLOCK_N / 2);
          const int c_half = col0 + warp_set * (BLOCK_N / 2);
          uint32_t ra[32], rb[32], rc[32], rd[32];
          bool ready = false, expired = false;
          uint32_t turns = 0;
          uint64_t t_first = 0;
#pragma unroll 1
          for (;;) {
            int r = 0;
            if (lane == 0) r = mbar_test_wait(tmem_full_bar, acc_phase) ? 1 : 0;
            ready = __shfl_sync(0xffffffffu, r, 0) != 0;
            if (ready) {
              tcgen05_fence_after();
              tmem_ld_32x32b_x32(t_half, ra);
              tmem_ld_32x32b_x32(t_half + 32, rb);
              tmem_ld_32x32b_x32(t_half + 64, rc);
              tmem_ld_32x32b_x32(t_half + 96, rd);
              tmem_ld_wait();
              break;
            }
            if ((++turns & 63u) == 0) {
              int stop = 0;
              if (lane == 0) {
                const uint64_t now = globaltimer_ns();
                if (t_first == 0) t_first = now;
                stop = (*abort_flag != 0 || now - t_first > kWaitLimitNs) ? 1 : 0;
              }
              if (__shfl_sync(0xffffffffu, stop, 0) != 0) { expired = true; break; }
            }
          }
          if (expired) {
            if (lane == 0) report_error(p, abort_flag, kDevTimeoutEpilogue, seg_idx, 0);
            break;
          }
          // The values sit in registers: tensor memory goes back before they are packed.
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) {
            if (kCtaGroup == 2) mbar_arrive_cluster(leader_tmem_empty);
            else mbar_arrive(tmem_empty_bar);
          }
          if (p.fuse) {
            fused_epilogue<32, false>(ra, p, row0 + row_in_cta, c_half);
            fused_epilogue<32, false>(rb, p, row0 + row_in_cta, c_half + 32);
            fused_epilogue<32, false>(rc, p, row0 + row_in_cta, c_half + 64);
            fused_epilogue<32, false>(rd, p, row0 + row_in_cta, c_half + 96);
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            packed[0][j] = pack_bf16x2(__uint_as_float(ra[2 * j]), __uint_as_float(ra[2 * j + 1]));
            packed[0][16 + j] = pack_bf16x2(__uint_as_float(rb[2 * j]), __uint_as_float(rb[2 * j + 1]));
            packed[0][32 + j] = pack_bf16x2(__uint_as_float(rc[2 * j]), __uint_as_float(rc[2 * j + 1]));
            packed[0][48 + j] = pack_bf16x2(__uint_as_float(rd[2 * j]), __uint_as_float(rd[2 * j + 1]));
          }
        }
        {
          constexpr int h = 1;
          const uint32_t t_half = taddr + h * BLOCK_N + warp_set * (BLOCK_N / 2);
          const int c_half = col0 + h * BLOCK_N + warp_set * (BLOCK_N / 2);
          {
#pragma unroll
            for (int bt = 0; bt < 2; ++bt) {
              uint32_t ra[32], rb[32];
              __syncwarp();
              tmem_ld_32x32b_x32(t_half + bt * 64, ra);
              tmem_ld_32x32b_x32(t_half + bt * 64 + 32, rb);
              tmem_ld_wait();
              if (bt == 1) {
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) {
                  if (kCtaGroup == 2) mbar_arrive_cluster(leader_tmem_empty + 8);
                  else mbar_arrive(tmem_empty_bar + 8);
                }
              }
              if (p.fuse) {
                fused_epilogue<32, false>(ra, p, row0 + row_in_cta, c_half + bt * 64);
                fused_epilogue<32, false>(rb, p, row0 + row_in_cta, c_half + bt * 64 + 32);
              }
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                packed[h][bt * 32 + j] =
                    pack_bf16x2(__uint_as_float(ra[2 * j]), __uint_as_float(ra[2 * j + 1]));
                packed[h][bt * 32 + 16 + j] =
                    pack_bf16x2(__uint_as_float(rb[2 * j]), __uint_as_float(rb[2 * j + 1]));
              }
            }
          }
        }
        released = true;
        const uint32_t sw = lane & 7u;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int h = i >> 1, b = i & 1;
          const int c = h * BLOCK_N + warp_set * (BLOCK_N / 2) + b * Cfg::EPI_COLS;
          const bool own_buf = (i == 0) || !ring_is_free;
          const uint32_t box_buf = own_buf
              ? buf : ring + static_cast<uint32_t>((warp - 2) * 3 + (i - 1)) * Cfg::SMEM_EPI_WARP_BUF;
          const uint32_t row_addr = box_buf + lane * 128u;
          if (own_buf && lane == 0) tma_store_wait_read<0>();   // the previous box has left it
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 8; ++j)
            st_shared_v4(row_addr + ((static_cast<uint32_t>(j) ^ sw) << 4),
                         packed[h][b * 32 + 4 * j + 0], packed[h][b * 32 + 4 * j + 1],
                         packed[h][b * 32 + 4 * j + 2], packed[h][b * 32 + 4 * j + 3]);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (my_row0 < p.Md && col0 + c < p.Nd) {
              if (p.l2_hints & 4) tma_store_2d_hint(&tmap_d, box_buf, col0 + c, my_row0, pol_d);
              else tma_store_2d(&tmap_d, box_buf, col0 + c, my_row0);
            }
            tma_store_commit();
          }
        }
      } else if (Cfg::kEpiMode == kEpiTmaStore) {
        const uint32_t warp_stage = epi_base + (warp - 2) * Cfg::kEpiBufs * Cfg::SMEM_EPI_WARP_BUF;
        const int my_row0 = row0 + quad * 32;
        // One-half tiles: this warp walks all BLOCK_N columns.  Two-half tiles: the two sets of
        // four warps split each half between them (128 columns = two boxes each) and do half 0
        // first, so that half 0 goes back to the MMA warp after two boxes, half 1 after four.
        constexpr int kBoxes = (Cfg::kNHalves == 1) ? BLOCK_N / Cfg::EPI_COLS : 4;
#pragma unroll 1
        for (int i = 0; i < kBoxes; ++i) {
          const int c = (Cfg::kNHalves == 1)
              ? i * Cfg::EPI_COLS
              : (i >> 1) * BLOCK_N + warp_set * (BLOCK_N / 2) + (i & 1) * Cfg::EPI_COLS;
          const bool last_of_accumulator = (Cfg::kNHalves == 1) ? (i == kBoxes - 1) : ((i & 1) == 1);
          const uint32_t buf = ring_is_free
              ? ring + static_cast<uint32_t>((warp - 2) * kBoxes + i) * Cfg::SMEM_EPI_WARP_BUF
              : warp_stage + (store_count % Cfg::kEpiBufs) * Cfg::SMEM_EPI_WARP_BUF;
          uint32_t r0[32], r1[32];
          __syncwarp();
          tmem_ld_32x32b_x32(taddr + c, r0);
          tmem_ld_32x32b_x32(taddr + c + 32, r1);
          tmem_ld_wait();
          if (last_of_accumulator) {
            // This warp's last columns of the accumulator are in registers: hand it back now,
            // before the conversion and the store of this box (one arrive per warp).
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
              const uint32_t which = (Cfg::kNHalves == 1) ? acc : static_cast<uint32_t>(i >> 1);
              if (kCtaGroup == 2) mbar_arrive_cluster(leader_tmem_empty + 8 * which);
              else mbar_arrive(tmem_empty_bar + 8 * which);
            }
            released = true;
          }
          // The store issued kEpiBufs boxes ago read from this buffer; make sure it is done.
          if (!ring_is_free && lane == 0) tma_store_wait_read<Cfg::kEpiBufs - 1>();
          __syncwarp();
          if (tile_partials != nullptr) {
            const float* base = tile_partials + static_cast<size_t>(c) * Cfg::TILE_M +
                                cta_rank * Cfg::BLOCK_M + row_in_cta;
            const size_t slot = static_cast<size_t>(BLOCK_N) * Cfg::TILE_M;
            // 16 columns at a time, one contributor in flight: this path is rare (cut last wave)
            // and must not cost the plain path registers.
            using Quarter = uint32_t(&)[16];
            sum_partials<16, 1>(reinterpret_cast<Quarter>(r0[0]), base, Cfg::TILE_M, slot,
                                seg.contrib, seg.n_contrib);
            sum_partials<16, 1>(reinterpret_cast<Quarter>(r0[16]), base + 16 * Cfg::TILE_M,
                                Cfg::TILE_M, slot, seg.contrib, seg.n_contrib);
            sum_partials<16, 1>(reinterpret_cast<Quarter>(r1[0]), base + 32 * Cfg::TILE_M,
                                Cfg::TILE_M, slot, seg.contrib, seg.n_contrib);
            sum_partials<16, 1>(reinterpret_cast<Quarter>(r1[16]), base + 48 * Cfg::TILE_M,
                                Cfg::TILE_M, slot, seg.contrib, seg.n_contrib);
          }
          if (p.fuse) {
            fused_epilogue<32>(r0, p, row0 + row_in_cta, col0 + c);
            fused_epilogue<32>(r1, p, row0 + row_in_cta, col0 + c + 32);
          }
          const uint32_t sw = lane & 7u;
          if (p.out32 != nullptr) {
            // fp32 result: a box is 32 rows x 32 columns (128 B per row), so each 64-column step
            // leaves as two boxes, r0 and r1, each through a staging buffer of its own: the
            // step's regular buffer and - for r1 - the other regular buffer (one-half tiles have
            // two per warp), or the next ring slot when the ring is free.
#pragma unroll
            for (int hb = 0; hb < 2; ++hb) {
              const uint32_t fbuf = ring_is_free
                  ? ring + static_cast<uint32_t>(((warp - 2) * kBoxes + i) * 2 + hb) * Cfg::SMEM_EPI_WARP_BUF
                  : warp_stage + static_cast<uint32_t>(hb) * Cfg::SMEM_EPI_WARP_BUF;
              // Buffer hb was last read by the store issued two groups ago: all but the most
              // recent group must have finished reading (hb == 0 was waited for above).
              if (!ring_is_free && hb == 1 && lane == 0) tma_store_wait_read<1>();
              __syncwarp();
              const uint32_t frow = fbuf + lane * 128u;
              const uint32_t* src = hb == 0 ? r0 : r1;
#pragma unroll
              for (int j = 0; j < 8; ++j)
                st_shared_v4(frow + ((static_cast<uint32_t>(j) ^ sw) << 4), src[4 * j + 0],
                             src[4 * j + 1], src[4 * j + 2], src[4 * j + 3]);
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                if (my_row0 < p.Md && col0 + c + 32 * hb < p.Nd)
                  tma_store_2d(&tmap_d, fbuf, col0 + c + 32 * hb, my_row0);
                tma_store_commit();
              }
            }
            ++store_count;
            continue;
          }
          const uint32_t row_addr = buf + lane * 128u;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            st_shared_v4(row_addr + ((static_cast<uint32_t>(j) ^ sw) << 4),
                         pack_bf16x2(__uint_as_float(r0[8 * j + 0]), __uint_as_float(r0[8 * j + 1])),
                         pack_bf16x2(__uint_as_float(r0[8 * j + 2]), __uint_as_float(r0[8 * j + 3])),
                         pack_bf16x2(__uint_as_float(r0[8 * j + 4]), __uint_as_float(r0[8 * j + 5])),
                         pack_bf16x2(__uint_as_float(r0[8 * j + 6]), __uint_as_float(r0[8 * j + 7])));
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            st_shared_v4(row_addr + ((static_cast<uint32_t>(j + 4) ^ sw) << 4),
                         pack_bf16x2(__uint_as_float(r1[8 * j + 0]), __uint_as_float(r1[8 * j + 1])),
                         pack_bf16x2(__uint_as_float(r1[8 * j + 2]), __uint_as_float(r1[8 * j + 3])),
                         pack_bf16x2(__uint_as_float(r1[8 * j + 4]), __uint_as_float(r1[8 * j + 5])),
                         pack_bf16x2(__uint_as_float(r1[8 * j + 6]), __uint_as_float(r1[8 * j + 7])));
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (my_row0 < p.Md && col0 + c < p.Nd) {
              if (p.l2_hints & 4) tma_store_2d_hint(&tmap_d, buf, col0 + c, my_row0, pol_d);
              else tma_store_2d(&tmap_d, buf, col0 + c, my_row0);
            }
            tma_store_commit();
          }
          ++store_count;
        }
      } else {
        bool stored = false;
        if constexpr (Cfg::kFlippable) {
          if (p.l2_hints & 64) {
            // Exchanged roles (see kFlippable): this lane holds, for ONE row of Y, the tile rows
            // 0 .. tile_rows-1 of one CTA of the pair in columns 0 .. tile_rows-1 - for a
            // transposed result that is tile_rows x 2 contiguous bytes.  The lanes stage their
            // rows in the idle ring as [half of the lanes][64 rows of Y][tile_rows], 16 bytes
            // at a time, and each warp hands its 32 rows to the TMA unit as one box.
            const int m_local = row_in_cta & 63;
            const uint32_t owner = quad >> 1;
            const uint32_t pitch = static_cast<uint32_t>(p.tile_rows) * 2u;
            const uint32_t dst = ring + owner * (64u * pitch) + static_cast<uint32_t>(m_local) * pitch;
#pragma unroll 1
            for (int c = 0; c < p.tile_rows; c += 32) {
              uint32_t r[32];
              __syncwarp();
              tmem_ld_32x32b_x32(taddr_tile + c, r);
              tmem_ld_wait();
#pragma unroll
              for (int v8 = 0; v8 < 4; ++v8) {
                if (c + 8 * v8 < p.tile_rows)
                  st_shared_v4(dst + static_cast<uint32_t>(c + 8 * v8) * 2u,
                               pack_bf16x2(__uint_as_float(r[8 * v8 + 0]), __uint_as_float(r[8 * v8 + 1])),
                               pack_bf16x2(__uint_as_float(r[8 * v8 + 2]), __uint_as_float(r[8 * v8 + 3])),
                               pack_bf16x2(__uint_as_float(r[8 * v8 + 4]), __uint_as_float(r[8 * v8 + 5])),
                               pack_bf16x2(__uint_as_float(r[8 * v8 + 6]), __uint_as_float(r[8 * v8 + 7])));
              }
            }
            // A warp's 32 rows of Y are a box of their own: no warp waits for another.
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              const int y = col0 + static_cast<int>(cta_rank) * 64 + static_cast<int>(quad & 1u) * 32;
              const int x = (tm * 2 + static_cast<int>(owner)) * p.tile_rows;
              if (x < p.Md && y < p.Nd)
                tma_store_2d(&tmap_d, dst - lane * pitch, x, y);
              tma_store_commit();
            }
            stored = true;
          }
        }
        if constexpr (Cfg::kMHalves == 2) {
          if (!stored && (p.l2_hints & 32)) {
            // Tall tile with a transposed bf16 result (rows of D contiguous in memory), the
            // decode case.  A tall tile is its CTA's only tile, so this walk is the exposed tail
            // of the launch, and it is bound by SM cycles, not by memory: stores from registers
            // took 700 cycles per 32-column step (four 16-byte store instructions, each eight
            // 64-byte pieces of eight different lines) against 155 for staging the step and 23
            // for reading it from tensor memory - the same count at any clock, and under the
            // power cap these shapes run at half the idle clock.  So the tile goes out as ONE
            // box: the operand ring is idle by now (every copy into it has been consumed by an
            // MMA that has completed), the four warps stage the whole tile there as
            // [column][tile_rows], a column being tile_rows x 2 contiguous bytes of the result,
            // and one thread hands it to the TMA unit, which clips it at the matrix edge.
            constexpr int kDC = Cfg::kDirectCols;
            const uint32_t pitch = static_cast<uint32_t>(p.tile_rows) * 2u;
#pragma unroll 1
            for (int mh = 0; mh < 2; ++mh) {
              const int r_in_tile = mh * Cfg::BLOCK_M + static_cast<int>(quad) * 32;
              if (r_in_tile >= p.tile_rows) continue;               // (warp-uniform)
              const bool mine = r_in_tile + static_cast<int>(lane) < p.tile_rows;
              const uint32_t taddr = taddr_tile + static_cast<uint32_t>(mh) * BLOCK_N;
              const uint32_t dst = ring + static_cast<uint32_t>(r_in_tile + static_cast<int>(lane)) * 2u;
#pragma unroll 1
              for (int c = 0; c < BLOCK_N; c += kDC) {
                uint32_t r[kDC];
                __syncwarp();
                if constexpr (kDC == 32) tmem_ld_32x32b_x32(taddr + c, r);
                else tmem_ld_32x32b_x16(taddr + c, r);
                tmem_ld_wait();
                if (p.fuse)
                  fused_epilogue<kDC>(r, p, row0_tile + r_in_tile + static_cast<int>(lane), col0 + c);
                if (mine) {
#pragma unroll
                  for (int j = 0; j < kDC; ++j)
                    st_shared_b16(dst + static_cast<uint32_t>(c + j) * pitch,
                                  __bfloat16_as_ushort(__float2bfloat16_rn(__uint_as_float(r[j]))));
                }
              }
            }
            // Writers fence their own writes towards the async proxy, then meet at a barrier of
            // the four epilogue warps; only the issuing thread has to wait there (bounded).
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(epi_sync_bar);
            if (warp == 2 && lane == 0) {
              if (mbar_wait(epi_sync_bar, static_cast<uint32_t>(seg_idx & 1), abort_flag)) {
                tma_store_2d(&tmap_d, ring, row0_tile, col0);
                tma_store_commit();
              } else {
                report_error(p, abort_flag, kDevTimeoutEpilogue, seg_idx, 7);
              }
            }
            stored = true;
          }
        }
        // Two M-halves: the same walk twice, 128 rows and BLOCK_N accumulator columns further on.
#pragma unroll 1
        for (int mh = 0; mh < (stored ? 0 : Cfg::kMHalves); ++mh) {
        const int row0 = row0_tile + mh * Cfg::BLOCK_M;
        const uint32_t taddr = taddr_tile + static_cast<uint32_t>(mh) * BLOCK_N;
        const int row = row0 + row_in_cta;
        __nv_bfloat16* out_row = p.out + static_cast<long long>(row) * p.out_stride_r;
        const bool vec_ok = (p.out_stride_c == 1) && ((p.out_stride_r & 7) == 0) &&
                            ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
        // Transposed result (rows of D are contiguous in memory): stage, then 16-byte stores.
        // An fp32 result is never staged: with one row per lane, the 32 lanes' stores of one
        // column are 128 contiguous bytes already.
        transposed = (p.out32 == nullptr) && (p.out_stride_r == 1) && ((p.out_stride_c & 7) == 0) &&
                     ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
        const uint32_t stg = (Cfg::kMHalves == 2 ? ring : epi_base) + (warp - 2) * Cfg::SMEM_EPI_T_WARP;
        // 32 columns per step where the tile has them: half as many dependent round trips to
        // the partials of a cut tile as with 16.
        constexpr int kDC = Cfg::kDirectCols;
        const int n0 = row0 + static_cast<int>(quad) * 32 + static_cast<int>(lane & 3u) * 8;
#pragma unroll 1
        for (int c = 0; c < BLOCK_N; c += kDC) {
          uint32_t r[kDC];
          // tcgen05.ld / wait::ld are .sync.aligned: every lane must arrive together.  Lanes
          // whose row is out of range skip the stores below and would otherwise run ahead.
          __syncwarp();
          if constexpr (kDC == 32) tmem_ld_32x32b_x32(taddr + c, r);
          else tmem_ld_32x32b_x16(taddr + c, r);
          tmem_ld_wait();
          if (tile_partials != nullptr) {
            sum_partials<kDC>(r, tile_partials + static_cast<size_t>(c) * Cfg::TILE_M +
                                     cta_rank * Cfg::BLOCK_M + row_in_cta,
                              Cfg::TILE_M, static_cast<size_t>(BLOCK_N) * Cfg::TILE_M, seg.contrib,
                              seg.n_contrib);
          }
          const int col = col0 + c;
          if (p.fuse) fused_epilogue<kDC>(r, p, row, col);
          if (transposed) {
            // (the __syncwarp in front of this step's tcgen05.ld is also what keeps these writes
            // behind the previous step's reads of the staging buffer)
#pragma unroll
            for (int j = 0; j < kDC; ++j)
              st_shared_b16(stg + static_cast<uint32_t>(j) * 64u + lane * 2u,
                            __bfloat16_as_ushort(__float2bfloat16_rn(__uint_as_float(r[j]))));
            __syncwarp();
            // Write-out of the staged step: column m of D is 32 contiguous bf16 (64 B) of the
            // result; four lanes cover one column, the warp covers eight columns per store.
#pragma unroll
            for (int m = static_cast<int>(lane >> 2); m < kDC; m += 8) {
              const int colm = col + m;
              if (colm >= p.Nd || n0 >= row_limit) continue;
              const long long off = static_cast<long long>(colm) * p.out_stride_c + n0;
              uint32_t v[4];
              ld_shared_v4(stg + static_cast<uint32_t>(m) * 64u + (lane & 3u) * 16u, v);
              if (n0 + 8 <= row_limit) {
                if (off + 8 > p.out_span) {
                  report_error(p, abort_flag, kDevBounds, seg_idx, 3);
                } else {
                  *reinterpret_cast<uint4*>(p.out + off) = make_uint4(v[0], v[1], v[2], v[3]);
                }
              } else {
                const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(v);
                for (int j = 0; j < 8 && n0 + j < row_limit; ++j) {
                  if (off + j < p.out_span) p.out[off + j] = e[j];
                }
              }
            }
          } else
          if (p.out32 != nullptr) {
            if (row < row_limit && col < p.Nd) {
              const int last_col = min(col + kDC - 1, p.Nd - 1);
              const long long last = static_cast<long long>(row) * p.out_stride_r +
                                     static_cast<long long>(last_col) * p.out_stride_c;
              float* out_row32 = p.out32 + static_cast<long long>(row) * p.out_stride_r;
              if (last >= p.out_span) {
                report_error(p, abort_flag, kDevBounds, seg_idx, 3);
              } else if (p.out_stride_c == 1 && (p.out_stride_r & 3) == 0 && col + kDC <= p.Nd &&
                         (reinterpret_cast<uintptr_t>(p.out32) & 15) == 0) {
#pragma unroll
                for (int v4 = 0; v4 < kDC / 4; ++v4)
                  *reinterpret_cast<uint4*>(out_row32 + col + 4 * v4) =
                      make_uint4(r[4 * v4 + 0], r[4 * v4 + 1], r[4 * v4 + 2], r[4 * v4 + 3]);
              } else {
#pragma unroll
                for (int j = 0; j < kDC; ++j) {
                  if (col + j < p.Nd)
                    out_row32[static_cast<long long>(col + j) * p.out_stride_c] = __uint_as_float(r[j]);
                }
              }
            }
          } else
          if (row < row_limit && col < p.Nd) {
            const int last_col = min(col + kDC - 1, p.Nd - 1);
            const long long last = static_cast<long long>(row) * p.out_stride_r +
                                   static_cast<long long>(last_col) * p.out_stride_c;
            if (last >= p.out_span) {
              report_error(p, abort_flag, kDevBounds, seg_idx, 3);
            } else
            if (vec_ok && col + kDC <= p.Nd) {
#pragma unroll
              for (int v8 = 0; v8 < kDC / 8; ++v8) {
                uint4 v;
                v.x = pack_bf16x2(__uint_as_float(r[8 * v8 + 0]), __uint_as_float(r[8 * v8 + 1]));
                v.y = pack_bf16x2(__uint_as_float(r[8 * v8 + 2]), __uint_as_float(r[8 * v8 + 3]));
                v.z = pack_bf16x2(__uint_as_float(r[8 * v8 + 4]), __uint_as_float(r[8 * v8 + 5]));
                v.w = pack_bf16x2(__uint_as_float(r[8 * v8 + 6]), __uint_as_float(r[8 * v8 + 7]));
                *reinterpret_cast<uint4*>(out_row + col + 8 * v8) = v;
              }
            } else {
#pragma unroll
              for (int j = 0; j < kDC; ++j) {
                if (col + j < p.Nd)
                  out_row[static_cast<long long>(col + j) * p.out_stride_c] =
                      __float2bfloat16_rn(__uint_as_float(r[j]));
              }
            }
          }
        }
        }
      }

      // Accumulator drained: hand it back to the MMA warp (one arrive per warp), unless the
      // store path already did so after its last tensor-memory load.
      __syncwarp();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0 && !released) {
        // (only reached by paths that did not hand the accumulator back earlier; two-half tiles
        // always do, in the store loop above)
        const uint32_t which = acc;
        if (kCtaGroup == 2) mbar_arrive_cluster(leader_tmem_empty + 8 * which);
        else mbar_arrive(tmem_empty_bar + 8 * which);
      }
      ++seg_idx;
    }
    if (it.failed && lane == 0) report_error(p, abort_flag, kDevTimeoutScheduler, seg_idx, 2);
    // Shared memory must outlive the stores' reads of it; their writes to global memory are
    // complete when the grid is, which is all a later kernel or copy can observe.
    if ((Cfg::kEpiMode == kEpiTmaStore || Cfg::kMHalves == 2) && lane == 0) tma_store_wait_read<0>();
    loop_timer.end();
    loop_timer.stamp(11);
    loop_timer.flush(6);
    wait_timer.flush(5);
    __syncwarp();
  }

  // ---------------------------------------------------------------- tear-down
  tcgen05_fence_before();
  if (kCtaGroup == 2) cluster_sync_all(); else __syncthreads();
  if (*abort_flag != 0) {
    // Let TMA boxes still in flight land in this CTA's shared memory before it is released.
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 1000000ull) __nanosleep(1000);
    if (kCtaGroup == 2) cluster_sync_all(); else __syncthreads();
  }
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc<1>(tmem_base, Cfg::kTmemCols);
  }
  if (threadIdx.x == 0) PhaseTimer(p).stamp(12);
}

// Second pass of a two-pass split-K launch.  When every tile of a launch is cut into the same
// number of k-chunks (few wide tiles under a long K: one chunk per CTA fills the machine where
// whole tiles would use a fraction of it), the GEMM kernel only publishes fp32 partials and this
// kernel, launched right behind it on the same stream, sums them in contributor order, applies
// the fused epilogue and stores D.  All SMs take part: a thread owns one row of a tile and eight
// consecutive columns, so every load of a partial is a coalesced 128-byte line per warp and the
// sums of different tiles, rows and column groups run in parallel - where a last-arriving
// contributor summing a 256 x 256 tile alone took longer than the product itself.
// Partial layout: [tile][contributor][column][row of the tile], as the GEMM kernel writes it.
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const __grid_constant__ GemmParams p, int tile_m, int block_n) {
  ptx::griddep_launch_dependents();
  ptx::griddep_wait();   // the partials of the GEMM kernel in front are complete and visible
  const int n = p.sk_splits;
  const int groups = block_n / 8;
  const long long per_tile = static_cast<long long>(tile_m) * groups;
  const long long total = per_tile * p.num_tiles;
  const size_t slot = static_cast<size_t>(block_n) * tile_m;
  for (long long item = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; item < total;
       item += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int tile = static_cast<int>(item / per_tile);
    const long long rest = item - tile * per_tile;
    const int g = static_cast<int>(rest / tile_m);
    const int r_in_tile = static_cast<int>(rest - static_cast<long long>(g) * tile_m);
    int tm, tn;
    tile_coords(p, tile, tm, tn);
    const int row = tm * tile_m + r_in_tile;
    const int col = tn * block_n + g * 8;
    if (row >= p.Md || col >= p.Nd) continue;
    const float* base = p.partials + static_cast<size_t>(tile) * p.max_contrib * slot +
                        static_cast<size_t>(g * 8) * tile_m + r_in_tile;
    float sum[8];
#pragma unroll 1
    for (int q0 = 0; q0 < n; q0 += 4) {
      float t[4][8];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (q0 + k < n) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            t[k][j] = __ldcg(base + static_cast<size_t>(q0 + k) * slot + static_cast<size_t>(j) * tile_m);
        }
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (q0 + k < n) {
#pragma unroll
          for (int j = 0; j < 8; ++j) sum[j] = (q0 + k == 0) ? t[k][j] : sum[j] + t[k][j];
        }
      }
    }
    uint32_t r[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = __float_as_uint(sum[j]);
    if (p.fuse) fused_epilogue<8>(r, p, row, col);
    // D is row-major here (the TMA-store kernels' layout) or any strided layout of the direct
    // kernels: eight columns of one row.
    const int last_col = min(col + 7, p.Nd - 1);
    const long long first = static_cast<long long>(row) * p.out_stride_r +
                            static_cast<long long>(col) * p.out_stride_c;
    const long long last = static_cast<long long>(row) * p.out_stride_r +
                           static_cast<long long>(last_col) * p.out_stride_c;
    if (last >= p.out_span || first < 0) {
      if (p.status != nullptr && atomicCAS(p.status, 0, kDevBounds) == 0) {
        p.status[1] = static_cast<int>(blockIdx.x);
        p.status[2] = -3;
        p.status[3] = 3;
        __threadfence_system();
      }
      continue;
    }
    const bool full = (col + 8 <= p.Nd) && (p.out_stride_c == 1);
    if (p.out32 != nullptr) {
      float* dst = p.out32 + first;
      if (full && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
        reinterpret_cast<uint4*>(dst)[0] = make_uint4(r[0], r[1], r[2], r[3]);
        reinterpret_cast<uint4*>(dst)[1] = make_uint4(r[4], r[5], r[6], r[7]);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (col + j < p.Nd) dst[static_cast<long long>(j) * p.out_stride_c] = __uint_as_float(r[j]);
      }
    } else {
      __nv_bfloat16* dst = p.out + first;
      if (full && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
        *reinterpret_cast<uint4*>(dst) = make_uint4(
            ptx::pack_bf16x2(__uint_as_float(r[0]), __uint_as_float(r[1])),
            ptx::pack_bf16x2(__uint_as_float(r[2]), __uint_as_float(r[3])),
            ptx::pack_bf16x2(__uint_as_float(r[4]), __uint_as_float(r[5])),
            ptx::pack_bf16x2(__uint_as_float(r[6]), __uint_as_float(r[7])));
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (col + j < p.Nd)
            dst[static_cast<long long>(j) * p.out_stride_c] = __float2bfloat16_rn(__uint_as_float(r[j]));
      }
    }
  }
}

// Self-test of the bounded-wait machinery: one warp waits, with the given limit, on an mbarrier
// that nothing will ever arrive on, and must come back with the limit expired, record the error
// like the GEMM roles do and exit normally.  No fault, no trap: the wait simply runs out.
__global__ void wait_expiry_selftest_kernel(GemmParams p, unsigned long long limit_ns,
                                            unsigned long long* waited_ns) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ int abort_word;
  const uint32_t bar_addr = ptx::smem_u32(&bar);
  if (threadIdx.x == 0) {
    abort_word = 0;
    ptx::mbar_init(bar_addr, 1);
    ptx::fence_barrier_init();
  }
  __syncthreads();
  const uint64_t t0 = ptx::globaltimer_ns();
  const bool completed = __all_sync(
      0xffffffffu, ptx::mbar_wait(bar_addr, 0, &abort_word, 0, limit_ns));
  const uint64_t t1 = ptx::globaltimer_ns();
  if (!completed && threadIdx.x == 0) {
    report_error(p, &abort_word, kDevTimeoutEpilogue, /*segment*/ -1, /*aux*/ -1);
    if (waited_ns != nullptr) *waited_ns = t1 - t0;
  }
}

}  // namespace neogemm
