// Persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   D[b, m, n] = epilogue( sum_k A[b, m, k] * B[b, n, k] )      (both operands K-major)
//
// which is the `out = a @ bt.T` convention of the reference's mm/addmm/bmm ops
// (ayla/gemm_jit.py:267-307): fp16/bf16 inputs, fp32 accumulation, one rounding
// to the output type at the end (ayla/passes/lower_to_ptx_template.py:134-149).
//
// One CTA = 11 warps:
//   warps 0, 10 TMA producers : global -> shared ring of STAGES (A 128x64, B BNx64) slabs, every
//                               other k-block each (one thread cannot start TMA loads fast enough)
//   warp 1      MMA issuer    : tcgen05.mma from shared into a TMEM accumulator;
//                               also owns the TMEM allocation
//   warps 2..9  epilogue      : TMEM -> registers -> (bias | activation | SiLU*up) -> round ->
//                               swizzled shared -> TMA store   (or direct stores for the
//                               transposed form and narrow cluster slices)
// The accumulator is double buffered in TMEM so the epilogue of one tile runs
// under the main loop of the next.  CTAs are persistent and walk a static,
// M-grouped raster over (batch, m-tile, n-tile, k-split) work units.
//
// CTA_GROUP == 2 pairs two CTAs (cluster of 2) on one 256-row tile: each CTA
// loads its own 128 rows of A and its own half of the B tile with ordinary TMA
// loads, the leader CTA issues tcgen05.mma.cta_group::2 for both.
//
// Launch overlap: the kernel runs its set-up, then executes griddepcontrol.wait before its first
// global access and griddepcontrol.launch_dependents right after, so that back-to-back launches
// issued with programmatic stream serialisation overlap set-up with the previous kernel's drain.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "sm100_prims.cuh"

namespace ayla_b200 {

enum : int { EPI_PLAIN = 0, EPI_BIAS = 1, EPI_SWIGLU = 2 };

// Error codes written to the device status word (first error wins).
enum : unsigned {
  ST_OK = 0,
  ST_TIMEOUT_EMPTY = 1,      // producer waited for a free ring slot
  ST_TIMEOUT_FULL = 2,       // MMA warp waited for operands
  ST_TIMEOUT_ACC_EMPTY = 3,  // MMA warp waited for a drained accumulator
  ST_TIMEOUT_ACC_FULL = 4,   // epilogue waited for a finished accumulator
  ST_BAD_SMEM_ALIGN = 5,
  ST_TIMEOUT_INBOX = 6,      // epilogue waited for the other k-splits' partial sums (cluster split-K)
};

// Division of a non-negative 32-bit value by a divisor fixed at launch: q = (n * mul) >> (32 + shift),
// with mul and shift worked out on the host (exact for n < 2^31).  A plain `/` on run-time values
// costs a dependent chain of some twenty instructions, and the schedule arithmetic at the head of
// every role has half a dozen of them in front of the first load.
struct FastDiv {
  uint32_t mul;    // 0: the divisor is 1
  uint32_t shift;
  __host__ __device__ static FastDiv make(uint32_t d) {
    FastDiv f{0u, 0u};
    if (d <= 1) return f;
    uint32_t l = 0;
    while ((1ull << l) < d) ++l;                       // ceil(log2 d) >= 1
    f.mul = static_cast<uint32_t>(((1ull << (31 + l)) / d) + 1);
    f.shift = l - 1;
    return f;
  }
#ifdef __CUDACC__
  __device__ __forceinline__ int div(int n) const {
    return mul == 0 ? n : static_cast<int>(__umulhi(static_cast<uint32_t>(n), mul) >> shift);
  }
#endif
};

struct KernelParams {
  int m, n, k;        // extents of the kernel's (row, column, depth) problem
  int batch;
  int m_tiles;        // tiles of 128*CTA_GROUP rows
  int n_tiles;        // tiles of the output tile width
  int k_blocks;       // ceil(k / 64)
  int splits;         // k-splits per split tile (1 = none)
  int kb_per_split;
  int split_from_tile;  // tiles with a linear index >= this are k-split; earlier tiles are whole
  int narrow_from_tile; // tiles >= this are done as two half-width units (no reduction needed)
  int cluster_split;    // S > 0: the S k-splits of a tile are the CTAs of one cluster and are
                        // summed through distributed shared memory (one tile per cluster)
  int stream_k;         // 1: every CTA takes an equal, contiguous share of all (tile, k-block) work
  int kb_per_cta;       // that share, in k-blocks
  uint32_t idesc_narrow; // instruction descriptor with N = BN / 2 for those units
  int total_units;    // batch * m_tiles * n_tiles * splits
  int group_m;        // raster: m-tiles per group
  int is_bf16;        // output / operand type: 1 bf16, 0 fp16
  uint32_t idesc;     // tcgen05 instruction descriptor
  uint32_t l2_hint_a; // 0 normal, 1 evict_first, 2 evict_last
  uint32_t l2_hint_b;
  const void* bias;   // [n] (or [m] when the output is transposed)
  void* out;          // used by the direct-store epilogues
  long long out_ld;   // leading dimension of `out` in elements (direct stores)
  long long out_batch_stride;
  float* ws;          // split-K partial slabs
  unsigned* counters; // split-K arrival counters, one per 128-row tile; zero between launches
  unsigned* status;   // optional device status word (may be null)
  unsigned long long timeout_ns;
  long long* trace;   // per-CTA cycle counters, written only by AYLA_B200_TRACE builds
  int debug_flags;    // bit 0: the producer issues no loads (exercises the bounded waits)
  int l2_prefetch;    // k-blocks the producer prefetches into L2 ahead of its shared-memory loads
  int early_prefetch; // k-blocks of the CTA's first unit asked into L2 before the dependency wait
  int early_operands; // which operands that prefetch covers: bit 0 the row operand, bit 1 the column operand
  FastDiv div_tiles_per_batch;  // by m_tiles * n_tiles
  FastDiv div_group_size;       // by group_m * n_tiles
  FastDiv div_group_m;          // by group_m
  FastDiv div_last_group_rows;  // by the row tiles of the last, partial raster group (m_tiles % group_m)
  FastDiv div_splits;           // by splits
  int ctas_per_unit_log2;       // log2(CTA_GROUP * cluster_split or 1)
  int stages;         // ring slots in use (<= the kernel's STAGES); fewer when the top of the ring region
                      // is set aside as the inbox of a cluster split-K launch
  uint32_t inbox_offset;  // cluster split-K: byte offset of the inbox from the start of shared memory
  uint32_t inbox_tx;      // bytes the inbox receives per launch
  int inbox_in_ring;      // 1: the inbox overlays ring slots that are in use, so partial sums may only be
                          // sent once every CTA of the cluster has finished its MMAs (one cluster barrier)
  const void* mul;    // optional gate, same shape and layout as `out`: out = act(...) * mul (activation variants)
  int mul_per_row;    // non-zero: `mul` holds one element per output row instead ([batch][rows])
  int act;            // activation applied to the fp32 result (after the bias) before rounding: ACT_*
  int tile_rows;      // swapped form: rows of the row operand per tile (8..128); 128 otherwise
  uint32_t stage_tx;  // bytes one ring stage receives (both CTAs of a pair together)
};

// Cycle accounting for tuning builds (-DAYLA_B200_TRACE): each role records the
// cycles it spent inside barrier waits and its total loop time.
#ifdef AYLA_B200_TRACE
// One point of a CTA's timeline: this SM's cycle counter, kept in shared memory until the CTA leaves
// (reading globaltimer costs some 0.15 us, and a store to global memory in flight delays the next
// release at cluster scope: both moved the times they were meant to measure).  Entry (slot 0) and exit
// (slot 5) also record globaltimer, in slots 32 and 33, which places the CTA's cycle counts on the time
// base all SMs share.
__device__ __forceinline__ void trace_stamp(long long* stamps, int slot) {
  stamps[slot] = clock64();
  if (slot == 0) stamps[32] = static_cast<long long>(global_timer_ns());
  if (slot == 5) stamps[33] = static_cast<long long>(global_timer_ns());
}
#endif
#ifdef AYLA_B200_TRACE
#define AYLA_TRACE_BEGIN long long tr_wait = 0, tr_wait2 = 0, tr_wait3 = 0, tr_tmp = 0; const long long tr_t0 = clock64();
#define AYLA_TRACE_WAIT(acc, stmt) tr_tmp = clock64(); stmt; acc += clock64() - tr_tmp;
#define AYLA_TRACE_END(slot)                                          \
  if (p.trace != nullptr && (threadIdx.x & 31) == 0) {                \
    p.trace[blockIdx.x * 16 + (slot) * 4 + 0] = tr_wait;              \
    p.trace[blockIdx.x * 16 + (slot) * 4 + 1] = tr_wait2;             \
    p.trace[blockIdx.x * 16 + (slot) * 4 + 2] = clock64() - tr_t0;    \
    p.trace[blockIdx.x * 16 + (slot) * 4 + 3] = tr_wait3;             \
  }
#else
#define AYLA_TRACE_BEGIN
#define AYLA_TRACE_WAIT(acc, stmt) stmt;
#define AYLA_TRACE_END(slot)
#endif

template <int BN_, int CTA_GROUP_, int EPI_, bool TRANS_OUT_, int STAGES_, bool ACT_ = false, bool LEAN_ = false>
struct GemmTraits {
  // LEAN: the kernel is compiled without the k-split epilogues (workspace and cluster forms) and
  // serves the launches that do not split k.  The unused code is never executed, yet it costs a
  // single-tile launch up to 1 us (instruction fetch), so those launches get a kernel without it.
  static constexpr bool LEAN = LEAN_;
  // ACT: the epilogue applies the activation named in the launch parameters.  A separate set of
  // instantiations, so that the plain kernels carry none of that code (compiled in as a run-time
  // branch it cost the output-bound bmm 5 %).
  static constexpr bool ACT = ACT_;
  static constexpr int BN = BN_;                // MMA N (accumulator columns)
  static constexpr int CTA_GROUP = CTA_GROUP_;
  static constexpr int EPI = EPI_;
  static constexpr bool TRANS_OUT = TRANS_OUT_;
  static constexpr int STAGES = STAGES_;
  static constexpr int BM = 128;                // rows per CTA
  static constexpr int BK = 64;                 // one 128-byte swizzle atom of 16-bit elements
  static constexpr int OUT_BN = (EPI == EPI_SWIGLU) ? BN / 2 : BN;  // output tile width
  static constexpr int B_ROWS = BN / CTA_GROUP; // B rows this CTA loads per stage
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = B_ROWS * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;  // one k-block of both operands
  // Consecutive k-blocks per slot of the ring (one barrier pair for all of them).  Handing a slot
  // from the loading warps to the MMA warp and back costs a few hundred cycles whatever the slot
  // holds; the MMAs of one k-block of a tile narrower than 256 columns take less than that, so
  // those tiles move two k-blocks per slot (measured on B200: M = 512, N = K = 4096 on 256 x 128
  // pair tiles 20.7 -> 17.9 us; M = 8, N = 14336 21.5 -> 19.3 us; four per slot gained nothing more).
  static constexpr int KB_PER_SLOT = (BN >= 256 || (BN == 192 && CTA_GROUP == 1)) ? 1 : 2;  // at least three slots
  static constexpr int SLOT_BYTES = KB_PER_SLOT * STAGE_BYTES;
  static constexpr int ACC_BUFS = 2;
  static constexpr int TMEM_COLS_NEEDED = ACC_BUFS * BN;
  static constexpr int TMEM_COLS = TMEM_COLS_NEEDED <= 32    ? 32
                                   : TMEM_COLS_NEEDED <= 64  ? 64
                                   : TMEM_COLS_NEEDED <= 128 ? 128
                                   : TMEM_COLS_NEEDED <= 256 ? 256
                                                             : 512;
  static constexpr int EPI_WARPS = 8;
  static constexpr int STORE_BUF_BYTES = 32 * 128;  // 32 rows x 64 columns of 16-bit
  static constexpr int STORE_BYTES = TRANS_OUT ? 0 : EPI_WARPS * STORE_BUF_BYTES;
  static constexpr int BIAS_BYTES = (EPI == EPI_BIAS && !TRANS_OUT) ? 2 * BN * 4 : 0;
  static constexpr int MISC_BYTES = 256;
#ifdef AYLA_B200_TRACE
  static constexpr int TRACE_BYTES = 40 * 8;  // the CTA's timeline stamps, copied out at exit
#else
  static constexpr int TRACE_BYTES = 0;
#endif
  static constexpr int SMEM_BYTES = STAGES * SLOT_BYTES + STORE_BYTES + BIAS_BYTES + MISC_BYTES + TRACE_BYTES;
  // Warps: 0 = first TMA producer, 1 = MMA issuer, 2..9 = epilogue, 10 = second TMA producer.
  static constexpr int PRODUCER2_WARP = 2 + EPI_WARPS;
  static constexpr int THREADS = 64 + EPI_WARPS * 32 + 32;
  static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "tcgen05 N extent");
  static_assert(B_BYTES % 1024 == 0, "B slab must keep the 1024-byte swizzle alignment");
  static_assert(EPI != EPI_SWIGLU || (BN == 256 && !TRANS_OUT), "SwiGLU uses the 2x128 layout");
  static_assert(TRANS_OUT || BN >= 64, "the TMA-store epilogue writes 64-column boxes");
  static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB shared-memory limit");
  static_assert((2 * STAGES + 2 * ACC_BUFS + 1) * 8 + 16 <= MISC_BYTES, "barrier area too small");
};

// A wait that gives up: polls the barrier, and every few thousand polls checks a
// CTA-wide abort flag and the global timer.  After a timeout the first error
// code is published, the abort flag is raised and every later wait in the CTA
// returns at once, so the kernel always terminates.
struct BoundedWait {
  volatile uint32_t* abort_flag;
  unsigned* status;
  unsigned long long timeout_ns;

  __device__ __forceinline__ bool aborted() const { return *abort_flag != 0; }

  __device__ __noinline__ void give_up(unsigned code) const {
    *abort_flag = 1;
    if (status != nullptr) atomicCAS(status, 0u, code | (blockIdx.x << 8));
  }

  __device__ __forceinline__ void wait(uint32_t bar, uint32_t parity, unsigned code) const {
    if (mbar_try_wait(bar, parity)) return;
    if (aborted()) return;
    uint64_t t0 = 0;
    uint32_t polls = 0;
    while (!mbar_try_wait(bar, parity)) {
      if ((++polls & 0x3F) == 0) {
        if (aborted()) return;
        const uint64_t now = global_timer_ns();
        if (t0 == 0) {
          t0 = now;
        } else if (now - t0 > timeout_ns) {
          give_up(code);
          return;
        }
      }
    }
  }
};

struct WorkUnit {
  int batch, m0, n0, kb0, kb1;
  int nsplit;      // CTAs contributing to this tile (1 = this unit owns the whole K range)
  int split;       // this unit's position among them (the order partials are summed in)
  int counter;     // arrival counter of the tile
  int slab0;       // static split: slab of contribution j is slab0 + j
  int tile;        // linear tile index
  bool is_split;
  bool is_narrow;  // covers only OUT_BN / 2 columns starting at n0
};

// Linear tile index -> (batch, m0, n0) through the M-grouped raster.
template <class T>
__device__ __forceinline__ void locate_tile(const KernelParams& p, int tile, int half, int cta_rank,
                                            WorkUnit& w) {
  const int tiles_per_batch = p.m_tiles * p.n_tiles;
  w.batch = p.div_tiles_per_batch.div(tile);
  const int t = tile - w.batch * tiles_per_batch;
  const int group_size = p.group_m * p.n_tiles;
  const int g = p.div_group_size.div(t);
  const int first_m = g * p.group_m;
  const bool full_group = p.m_tiles - first_m >= p.group_m;
  const int rows_in_group = full_group ? p.group_m : p.m_tiles - first_m;
  const int r = t - g * group_size;
  const int n_t = full_group ? p.div_group_m.div(r) : p.div_last_group_rows.div(r);
  const int m_t = first_m + (r - n_t * rows_in_group);
  // The swapped form may use fewer than 128 rows of its tile (tile_rows).
  w.m0 = T::TRANS_OUT ? m_t * p.tile_rows : (m_t * T::CTA_GROUP + cta_rank) * T::BM;
  w.n0 = n_t * T::OUT_BN + half * (T::OUT_BN / 2);
  w.tile = tile;
}

// The sequence of work units of one CTA (of one CTA pair when CTA_GROUP == 2).
//  * static schedule: units cta, cta + G, cta + 2G, ... of a list of whole tiles,
//    optionally followed by k-split tiles or half-width tiles;
//  * stream-K schedule: the contiguous range [cta * kb_per_cta, (cta + 1) * kb_per_cta) of
//    the (tile, k-block) sequence, cut at tile boundaries.  A tile cut between CTAs is
//    finished by whichever contributor arrives last, summing in CTA order.
template <class T>
struct UnitCursor {
  const KernelParams& p;
  const int cta_rank;
  const int cta, num_ctas;
  const int split_rank;  // cluster split-K: this CTA's k-split
  int unit;      // static
  int pos, end;  // stream-K, in k-blocks of the whole problem

  __device__ UnitCursor(const KernelParams& p_, int cta_, int num_ctas_, int cta_rank_, int split_rank_ = 0)
      : p(p_), cta_rank(cta_rank_), cta(cta_), num_ctas(num_ctas_), split_rank(split_rank_), unit(cta_) {
    const long long total = static_cast<long long>(p.total_units);  // stream-K: total k-blocks
    const long long b = static_cast<long long>(cta_) * p.kb_per_cta;
    const long long e = b + p.kb_per_cta;
    pos = static_cast<int>(b < total ? b : total);
    end = static_cast<int>(e < total ? e : total);
  }

  __device__ __forceinline__ bool next(WorkUnit& w) {
    if (p.stream_k) {
      if (pos >= end) return false;
      const int tile = pos / p.k_blocks;
      const int tile_kb0 = tile * p.k_blocks;
      locate_tile<T>(p, tile, 0, cta_rank, w);
      w.is_narrow = false;
      w.kb0 = pos - tile_kb0;
      w.kb1 = min(p.k_blocks, end - tile_kb0);
      pos = tile_kb0 + w.kb1;
      const int first_cta = tile_kb0 / p.kb_per_cta;
      const int last_cta = (tile_kb0 + p.k_blocks - 1) / p.kb_per_cta;
      w.nsplit = last_cta - first_cta + 1;
      w.split = cta - first_cta;
      w.is_split = w.nsplit > 1;
      w.counter = first_cta * T::CTA_GROUP + cta_rank;
      w.slab0 = 0;
      return true;
    }
    if (unit >= p.total_units) return false;
    int tile, half = 0;
    w.is_narrow = false;
    w.is_split = false;
    w.nsplit = 1;
    w.split = 0;
    if (p.cluster_split > 0) {
      // One tile per cluster; this CTA's share of K is its rank in the cluster.
      tile = unit;
      w.split = split_rank;
      w.nsplit = p.cluster_split;
      w.is_split = true;
    } else if (unit >= p.narrow_from_tile) {
      // Two half-width units per tile (never combined with k-splitting).
      const int u = unit - p.narrow_from_tile;
      tile = p.narrow_from_tile + (u >> 1);
      half = u & 1;
      w.is_narrow = true;
    } else if (unit < p.split_from_tile) {
      tile = unit;
    } else {
      const int u = unit - p.split_from_tile;
      const int q = p.div_splits.div(u);
      tile = p.split_from_tile + q;
      w.split = u - q * p.splits;
      w.nsplit = p.splits;
      w.is_split = p.splits > 1;
    }
    locate_tile<T>(p, tile, half, cta_rank, w);
    if (w.is_split) {
      w.kb0 = w.split * p.kb_per_split;
      w.kb1 = min(p.k_blocks, w.kb0 + p.kb_per_split);
    } else {
      w.kb0 = 0;
      w.kb1 = p.k_blocks;
    }
    // Index of this CTA's 128-row tile among the split tiles (slabs and counters).
    w.counter = (tile - p.split_from_tile) * T::CTA_GROUP + cta_rank;
    w.slab0 = w.counter * p.splits;
    unit += num_ctas;
    return true;
  }

  // True when at least n (1 or 2) more units follow the one `next` returned last.
  __device__ __forceinline__ bool follows(int n) const {
    if (p.stream_k) {
      if (pos >= end) return false;
      return n <= 1 || (pos / p.k_blocks + 1) * p.k_blocks < end;
    }
    return unit + (n - 1) * num_ctas < p.total_units;
  }

  // Slab that holds contribution j (0 <= j < nsplit) to the tile of unit w.
  __device__ __forceinline__ int slab_of(const WorkUnit& w, int j) const {
    if (!p.stream_k) return w.slab0 + j;
    // Each CTA owns two slabs: one for the first segment of its range, one for its last.
    const int first_cta = (w.tile * p.k_blocks) / p.kb_per_cta;
    const int c = first_cta + j;
    const int starts_in_tile = (c * p.kb_per_cta >= w.tile * p.k_blocks) ? 1 : 0;
    return (2 * c + (starts_in_tile ? 0 : 1)) * T::CTA_GROUP + cta_rank;
  }
};

__device__ __forceinline__ uint32_t pack2(float lo, float hi, int is_bf16) {
  if (is_bf16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float2 unpack2(uint32_t v, int is_bf16) {
  if (is_bf16) return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v));
  return __half22float2(*reinterpret_cast<const __half2*>(&v));
}

__device__ __forceinline__ float load_elem(const void* base, long long i, int is_bf16) {
  if (is_bf16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[i]);
  return __half2float(reinterpret_cast<const __half*>(base)[i]);
}

__device__ __forceinline__ void store_elem(void* base, long long i, float v, int is_bf16) {
  if (is_bf16) {
    reinterpret_cast<__nv_bfloat16*>(base)[i] = __float2bfloat16_rn(v);
  } else {
    reinterpret_cast<__half*>(base)[i] = __float2half_rn(v);
  }
}

// silu(g) * u on fp32 accumulators, before the single rounding; same order of
// operations as the reference's silu lowering (x * 1/(1+2^(-x*log2e)),
// ayla/passes/lower_to_ptx_template.py:296-315).
__device__ __forceinline__ float silu_mul(float g, float u) {
  const float e = exp2f(-g * 1.4426950408889634f);
  return __fdividef(g, 1.0f + e) * u;
}

// Activations of the fused epilogue, evaluated on the fp32 accumulator before the single
// rounding to the output type, as the reference's fused sigmoid is
// (ayla/passes/lower_to_ptx_template.py:84-113).
enum : int { ACT_NONE = 0, ACT_RELU = 1, ACT_SIGMOID = 2, ACT_SILU = 3, ACT_GELU = 4, ACT_GELU_TANH = 5 };

__device__ __forceinline__ float apply_act(float x, int act) {
  switch (act) {
    case ACT_RELU:
      return fmaxf(x, 0.0f);
    case ACT_SIGMOID:
      return __fdividef(1.0f, 1.0f + exp2f(-x * 1.4426950408889634f));
    case ACT_SILU:
      return __fdividef(x, 1.0f + exp2f(-x * 1.4426950408889634f));
    case ACT_GELU:
      return 0.5f * x * (1.0f + erff(x * 0.7071067811865476f));
    case ACT_GELU_TANH: {
      const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      return 0.5f * x * (1.0f + tanhf(u));
    }
    default:
      return x;
  }
}

// The same over the first COUNT values of a thread's chunk, with the choice of activation taken
// once outside the loop: each activation gets its own short unrolled loop, so a launch executes
// one contiguous piece of code instead of stepping through a switch per element.
template <int COUNT, int N>
__device__ __forceinline__ void apply_act_chunk(float (&v)[N], int act) {
  static_assert(COUNT <= N, "chunk larger than its array");
  switch (act) {
    case ACT_RELU:
#pragma unroll
      for (int j = 0; j < COUNT; ++j) v[j] = apply_act(v[j], ACT_RELU);
      break;
    case ACT_SIGMOID:
#pragma unroll
      for (int j = 0; j < COUNT; ++j) v[j] = apply_act(v[j], ACT_SIGMOID);
      break;
    case ACT_SILU:
#pragma unroll
      for (int j = 0; j < COUNT; ++j) v[j] = apply_act(v[j], ACT_SILU);
      break;
    case ACT_GELU:
#pragma unroll
      for (int j = 0; j < COUNT; ++j) v[j] = apply_act(v[j], ACT_GELU);
      break;
    case ACT_GELU_TANH:
#pragma unroll
      for (int j = 0; j < COUNT; ++j) v[j] = apply_act(v[j], ACT_GELU_TANH);
      break;
    default:
      break;
  }
}

__device__ __forceinline__ uint64_t make_policy(uint32_t hint) {
  if (hint == 1) return policy_evict_first();
  if (hint == 2) return policy_evict_last();
  return policy_evict_normal();
}

template <class T>
__global__ void __launch_bounds__(T::THREADS, 1)
gemm_sm100_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                  const __grid_constant__ CUtensorMap tm_b2, const __grid_constant__ CUtensorMap tm_d,
                  const KernelParams p) {
#if defined(__CUDA_ARCH_FEAT_SM100_ALL) || defined(__CUDA_ARCH_FEAT_SM101_ALL)
  constexpr int BN = T::BN;
  constexpr int CG = T::CTA_GROUP;
  constexpr int STAGES = T::STAGES;

  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* smem_store = smem + STAGES * T::SLOT_BYTES;
  float* smem_bias = reinterpret_cast<float*>(smem_store + T::STORE_BYTES);
  uint8_t* smem_misc = smem_store + T::STORE_BYTES + T::BIAS_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_misc);
  // barrier layout: full[STAGES], empty[STAGES], acc_full[2], acc_empty[2], inbox
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + STAGES * 8;
  const uint32_t bar_acc_full = bar_empty + STAGES * 8;
  const uint32_t bar_acc_empty = bar_acc_full + T::ACC_BUFS * 8;
  const uint32_t bar_inbox = bar_acc_empty + T::ACC_BUFS * 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2 * T::ACC_BUFS + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile uint32_t* last_flag = tmem_slot + 2;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
#ifdef AYLA_B200_TRACE
  // Timeline of this CTA in cycles of its SM (see trace_stamp).
  // Slots: 0 entry, 1 set-up done, 2 first operands landed, 3 last MMA committed, 4 epilogue done, 5 exit,
  // 6/7 cluster split-K barriers, 8 SM id, 9-11 a quarter / half / three quarters of the CTA's first unit
  // issued, 12 first TMA load issued, 13 epilogue saw the first finished accumulator, 14 the preceding
  // launch is complete (dependency wait returned), 15 split-k parts sent, 16 first accumulator chunk in
  // registers, 17 last output chunk handed to the store path, 18-21 the first warp's 64-column groups done,
  // 22/23 its first two chunks staged, 24 staging published to the async proxy, 25 bulk store issued,
  // 26 split-k: own partial of the first chunk in registers, 27 that chunk summed.
  long long* stamps = (p.trace != nullptr) ? reinterpret_cast<long long*>(smem_misc + T::MISC_BYTES) : nullptr;
  if (stamps != nullptr && threadIdx.x == 0) {
    for (int i = 0; i < 40; ++i) stamps[i] = 0;
    trace_stamp(stamps, 0);
    uint32_t smid;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    stamps[8] = static_cast<long long>(smid) + 1;
  }
#endif
  // A CTA pair is two CTAs whose ranks in the cluster differ in the last bit; with cluster
  // split-K a cluster holds several pairs, so the leader is the even rank of the pair,
  // not rank 0 of the cluster.
  const uint32_t cluster_rank = (CG == 2) ? cluster_ctarank() : 0u;
  const uint32_t cta_rank = cluster_rank & 1u;
  const uint32_t pair_base = cluster_rank & ~1u;
  const uint16_t pair_mask = static_cast<uint16_t>(0x3u << pair_base);
  const bool is_leader = cta_rank == 0;

  const BoundedWait bw{abort_flag, p.status, p.timeout_ns};
  // Cluster split-K: the cluster holds `csk` CTAs (CTA pairs when CG == 2), one per k-split
  // of the cluster's tile.
  const int csk = (T::EPI != EPI_SWIGLU && !T::LEAN) ? p.cluster_split : 0;
  constexpr int group = T::KB_PER_SLOT;  // k-blocks per ring slot
  const int n_stages = p.stages;         // ring slots in use

  if (threadIdx.x == 0) {
    // Descriptor fetches first: they overlap the barrier set-up below.
    prefetch_tensormap(&tm_a);
    prefetch_tensormap(&tm_b);
    if constexpr (T::EPI == EPI_SWIGLU) prefetch_tensormap(&tm_b2);
    if constexpr (!T::TRANS_OUT) prefetch_tensormap(&tm_d);
    *abort_flag = 0;
    *last_flag = 0;
    if ((smem_u32(smem) & 1023u) != 0) bw.give_up(ST_BAD_SMEM_ALIGN);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + s * 8, 1);
      mbar_init(bar_empty + s * 8, 1);
    }
    for (int b = 0; b < T::ACC_BUFS; ++b) {
      mbar_init(bar_acc_full + b * 8, 1);
      mbar_init(bar_acc_empty + b * 8, T::EPI_WARPS * CG);
    }
    mbar_init(bar_inbox, 1);
    // The inbox is used once per launch (one tile per cluster): announce its bytes now, before any
    // CTA of the cluster can send.
    if (csk > 0) mbar_arrive_expect_tx(bar_inbox, p.inbox_tx);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc<CG>(smem_u32(tmem_slot), T::TMEM_COLS);
    tmem_relinquish<CG>();
  }
  tc_fence_before_sync();
  if constexpr (CG == 1) {
    // The producer warp needs only the barriers its own lane 0 has just initialised, so
    // it announces them and starts loading at once; everyone else also waits for the
    // TMEM allocation.
    if (warp == 0) {
      __syncwarp();
      __threadfence_block();
      named_bar_arrive(3, T::THREADS);
    } else {
      named_bar_sync(3, T::THREADS);
    }
    // Cluster split-K: the other CTAs of the cluster will write into this CTA's inbox and credit
    // its inbox barrier.  Every thread announces here that the barrier exists and collects the
    // same announcement of the whole cluster later, where it costs nothing: the loading and
    // issuing warps after their loops, the epilogue warps just before they send.
    if (csk > 0) cluster_arrive_relaxed();
  } else {
    __syncthreads();
    // Both CTAs' barriers must exist before either one signals the other (their initialisation
    // was published by fence_mbar_init above).
    cluster_arrive_relaxed();
    cluster_wait();
  }
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
#ifdef AYLA_B200_TRACE
  if (stamps != nullptr && threadIdx.x == 32) trace_stamp(stamps, 1);
#endif

  // Everything above touched only this launch's own shared memory, TMEM and parameters, and so
  // does each role's own preparation below (schedule arithmetic, cache policies, L2 prefetches,
  // which move no data into this kernel).  A role executes griddepcontrol.wait itself right
  // before its first read or write of global memory: the launch that precedes this one in the
  // stream is then complete (a no-op unless the launch was allowed to start early).  The next
  // launch may begin its own set-up on SMs that fall idle from here on.
  grid_launch_dependents();

  const int csk_rank = csk > 0 ? static_cast<int>(cluster_ctarank()) / CG : 0;
  const int first_unit = static_cast<int>(blockIdx.x >> p.ctas_per_unit_log2);
  const int unit_stride = static_cast<int>(gridDim.x >> p.ctas_per_unit_log2);

  // The producer and MMA warps run their loops with all 32 lanes (addresses,
  // coordinates and descriptors are warp-uniform, which lets the compiler keep them
  // in uniform registers) and only one elected lane issues the asynchronous
  // instructions.
  if (warp == 0 || warp == T::PRODUCER2_WARP) {
    // ------------------------------------------------------------ TMA producers
    // Two warps, each filling every other ring slot (both operands of it).  One thread can start
    // a TMA tile load only every ~215 cycles, whatever the size of the box (measured on B200: 8
    // to 128 rows of 128 bytes alike; two threads of different warps reach twice the rate).  With
    // two loads per k-block a single producer holds every schedule to ~430 cycles per k-block:
    // no tile narrower than 256 x 256 per CTA pair could feed its MMAs (256 x 128 pairs ran at
    // 433 cycles per k-block against 256 tensor cycles) and a small-M weight stream could not go
    // faster than one 16 KB slab per 430 cycles per SM.
    // With debug bit 0 set nothing is ever loaded: the MMA warp's wait for operands runs
    // out and the launch ends with ST_TIMEOUT_FULL in the status word.
    const uint32_t prod_id = (warp == 0) ? 0u : 1u;
    uint32_t slot_count = 0;  // ring slots this CTA has used so far, over all its units
    const bool issuer = elect_one() && (p.debug_flags & 1) == 0;
    const uint64_t pol_a = make_policy(p.l2_hint_a);
    const uint64_t pol_b = make_policy(p.l2_hint_b);
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t full_bar0 = (CG == 2) ? map_to_cta(bar_full, pair_base) : bar_full;
    uint32_t stage = 0, phase = 0;
#ifdef AYLA_B200_TRACE
    bool first_issue_stamped = false;
#endif
    AYLA_TRACE_BEGIN
    UnitCursor<T> cursor(p, first_unit, unit_stride, cta_rank, csk_rank);
    WorkUnit w;
    bool dependency_met = false;
    while (cursor.next(w)) {
      if (bw.aborted()) break;
      // A narrow unit needs only the first half of each CTA's B slab; the full box is
      // still loaded (its tail is ignored by the narrower MMA).
      const int b_row = (T::EPI == EPI_SWIGLU)
                            ? w.n0
                            : w.n0 + static_cast<int>(cta_rank) * (w.is_narrow ? T::B_ROWS / 2 : T::B_ROWS);
      const int b_batch = (T::EPI == EPI_SWIGLU) ? 0 : w.batch;
      const CUtensorMap* tm_b_mine = &tm_b;
      if constexpr (T::EPI == EPI_SWIGLU && CG == 2) tm_b_mine = is_leader ? &tm_b : &tm_b2;
      auto prefetch_l2 = [&](int kb) {
        tma_prefetch_l2_3d(&tm_a, kb * T::BK, w.m0, w.batch);
        tma_prefetch_l2_3d(tm_b_mine, kb * T::BK, b_row, b_batch);
        if constexpr (T::EPI == EPI_SWIGLU && CG == 1) tma_prefetch_l2_3d(&tm_b2, kb * T::BK, b_row, 0);
      };
      const int pf = p.l2_prefetch;
      if (!dependency_met) {
        // Before the preceding launch is known to be complete nothing may be read into this
        // kernel, but its first operands may be asked into L2 (a prefetch delivers no data, and
        // L2 stays coherent with whatever that launch still writes): the loads issued after the
        // wait then find them there instead of paying the DRAM latency with an empty ring.
        // A prefetch occupies the issuing thread as long as a load does, so each producer asks for
        // the k-blocks it will load itself, and only for the operands worth it (the large ones).
        if (issuer) {
          for (int i = 0; i < p.early_prefetch && w.kb0 + i < w.kb1; ++i) {
            if (((slot_count + static_cast<uint32_t>(i / group)) & 1u) != prod_id) continue;
            const int kb = w.kb0 + i;
            if (p.early_operands & 1) tma_prefetch_l2_3d(&tm_a, kb * T::BK, w.m0, w.batch);
            if (p.early_operands & 2) {
              tma_prefetch_l2_3d(tm_b_mine, kb * T::BK, b_row, b_batch);
              if constexpr (T::EPI == EPI_SWIGLU && CG == 1) tma_prefetch_l2_3d(&tm_b2, kb * T::BK, b_row, 0);
            }
          }
        }
        grid_dependency_wait();
        dependency_met = true;
#ifdef AYLA_B200_TRACE
        if (stamps != nullptr && lane == 0 && prod_id == 0) trace_stamp(stamps, 14);
#endif
      }
      if (issuer && pf > 0 && prod_id == 0) {
        for (int kb = w.kb0; kb < w.kb1 && kb < w.kb0 + pf; ++kb) prefetch_l2(kb);
      }
      // One ring slot holds `group` consecutive k-blocks (one barrier pair for all of them): the
      // hand-over of a slot between the warps costs a couple of hundred cycles whatever it holds.
      for (int kb = w.kb0; kb < w.kb1; kb += group, ++slot_count) {
        const bool mine = (slot_count & 1u) == prod_id;  // the other producer fills the slots in between
        if (mine) {
          AYLA_TRACE_WAIT(tr_wait, bw.wait(bar_empty + stage * 8, phase ^ 1, ST_TIMEOUT_EMPTY))
        }
#ifdef AYLA_B200_TRACE
        if (issuer && mine && stamps != nullptr && !first_issue_stamped && prod_id == 0) {
          trace_stamp(stamps, 12);
          first_issue_stamped = true;
        }
#endif
        if (issuer && mine) {
          const uint32_t full_bar = full_bar0 + stage * 8;
          const int blocks = min(group, w.kb1 - kb);  // a unit may end in the middle of a slot
#ifdef AYLA_B200_TUNE
          if (p.debug_flags & 4) {  // tuning builds: hand the slot over without loading anything
            if (is_leader) mbar_arrive(bar_full + stage * 8);
          } else
#endif
          {
            if (is_leader) mbar_arrive_expect_tx(bar_full + stage * 8, p.stage_tx * static_cast<uint32_t>(blocks));
#pragma unroll
            for (int g = 0; g < group; ++g) {
              if (g < blocks) {
                const uint32_t sa = smem_base + stage * T::SLOT_BYTES + g * T::STAGE_BYTES;
                const uint32_t sb = sa + T::A_BYTES;
                const int k0 = (kb + g) * T::BK;
                tma_load_3d<CG>(sa, &tm_a, full_bar, k0, w.m0, w.batch, pol_a);
                if constexpr (T::EPI == EPI_SWIGLU && CG == 1) {
                  // Accumulator columns [0,128) = gate, [128,256) = up.
                  tma_load_3d<CG>(sb, &tm_b, full_bar, k0, b_row, 0, pol_b);
                  tma_load_3d<CG>(sb + T::B_BYTES / 2, &tm_b2, full_bar, k0, b_row, 0, pol_b);
                } else {
                  // Pair + SwiGLU: the leader's half of the B tile is gate, the peer's half is up.
                  tma_load_3d<CG>(sb, tm_b_mine, full_bar, k0, b_row, b_batch, pol_b);
                }
                if (pf > 0 && kb + g + pf < w.kb1) prefetch_l2(kb + g + pf);
              }
            }
          }
        }
        if (++stage == n_stages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
#ifdef AYLA_B200_TRACE
    if (prod_id == 0) {
      AYLA_TRACE_END(0)
    }
#endif
    if (CG == 1 && csk > 0) cluster_wait();
    if (csk > 0 && p.inbox_in_ring) {
      // A cluster barrier counts every thread of the cluster: keep step with the one the
      // epilogue warps use before they send their partial tiles.
      cluster_arrive_relaxed();
      cluster_wait();
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (is_leader) {
      const bool issuer = elect_one();
      const uint64_t desc_a0 = umma_smem_desc_sw128(smem_u32(smem));
      const uint64_t desc_b0 = umma_smem_desc_sw128(smem_u32(smem) + T::A_BYTES);
      const uint32_t idesc = p.idesc;
      uint32_t stage = 0, phase = 0;
      uint32_t acc = 0, acc_phase = 0;
#ifdef AYLA_B200_TRACE
      bool first_operands_stamped = false;
      bool first_unit_of_cta = true;
      long long tr_fence = 0, tr_issue = 0, tr_commit = 0, tr_iters = 0;
#endif
      AYLA_TRACE_BEGIN
      UnitCursor<T> cursor(p, first_unit, unit_stride, 0, csk_rank);
      WorkUnit w;
      while (cursor.next(w)) {
        if (bw.aborted()) break;
        AYLA_TRACE_WAIT(tr_wait2, bw.wait(bar_acc_empty + acc * 8, acc_phase ^ 1, ST_TIMEOUT_ACC_EMPTY))
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * BN;
        const uint32_t unit_idesc = w.is_narrow ? p.idesc_narrow : idesc;
        const int nkb = w.kb1 - w.kb0;
        for (int i = 0; i < nkb; i += group) {
          AYLA_TRACE_WAIT(tr_wait, bw.wait(bar_full + stage * 8, phase, ST_TIMEOUT_FULL))
#ifdef AYLA_B200_TRACE
          if (stamps != nullptr && lane == 0 && !first_operands_stamped) {
            trace_stamp(stamps, 2);
            first_operands_stamped = true;
          }
          if (stamps != nullptr && lane == 0 && first_unit_of_cta) {
            const int span = nkb, done = i;
            for (int qd = 1; qd <= 3; ++qd) {
              if (span >= 4 && done <= qd * span / 4 && qd * span / 4 < done + group) {
                trace_stamp(stamps, 8 + qd);
              }
            }
          }
#endif
#ifdef AYLA_B200_TRACE
          const long long tr_a = clock64();
#endif
          tc_fence_after_sync();
#ifdef AYLA_B200_TRACE
          const long long tr_b = clock64();
          tr_fence += tr_b - tr_a;
#endif
          if (issuer) {
            // Slot offset and the +32 bytes per 16-element K step, both in the descriptor's
            // 16-byte address units.
            const uint32_t slot_off = stage * (T::SLOT_BYTES >> 4);
            const int blocks = min(group, nkb - i);  // a unit may end in the middle of a slot
#ifdef AYLA_B200_TUNE
            if ((p.debug_flags & 8) == 0)
#endif
            {
#pragma unroll
              for (int g = 0; g < group; ++g) {
                if (g < blocks) {
#pragma unroll
                  for (int k4 = 0; k4 < T::BK / 16; ++k4) {
                    const uint32_t off = slot_off + g * (T::STAGE_BYTES >> 4) + 2 * k4;
                    umma_f16<CG>(tmem_d, desc_a0 + off, desc_b0 + off, unit_idesc, (i + g > 0 || k4 > 0) ? 1u : 0u);
                  }
                }
              }
            }
#ifdef AYLA_B200_TRACE
            const long long tr_c = clock64();
            tr_issue += tr_c - tr_b;
#endif
#ifdef AYLA_B200_TUNE
            if (p.debug_flags & 16) {
              mbar_arrive(bar_empty + stage * 8);
            } else
#endif
            if constexpr (CG == 1) {
              umma_commit_1cta(bar_empty + stage * 8);
            } else {
              umma_commit_2cta(bar_empty + stage * 8, pair_mask);
            }
            if (i + group >= nkb) {
              if constexpr (CG == 1) {
                umma_commit_1cta(bar_acc_full + acc * 8);
              } else {
                umma_commit_2cta(bar_acc_full + acc * 8, pair_mask);
              }
            }
#ifdef AYLA_B200_TRACE
            tr_commit += clock64() - tr_c;
            ++tr_iters;
#endif
          }
          if (++stage == n_stages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (++acc == T::ACC_BUFS) {
          acc = 0;
          acc_phase ^= 1;
        }
#ifdef AYLA_B200_TRACE
        first_unit_of_cta = false;
#endif
      }
      AYLA_TRACE_END(1)
#ifdef AYLA_B200_TRACE
      if (stamps != nullptr && lane == 0) trace_stamp(stamps, 3);
      if (p.trace != nullptr && issuer) {
        p.trace[blockIdx.x * 16 + 12] = tr_fence;
        p.trace[blockIdx.x * 16 + 13] = tr_issue;
        p.trace[blockIdx.x * 16 + 14] = tr_commit;
        p.trace[blockIdx.x * 16 + 15] = tr_iters;
      }
#endif
    }
    if (CG == 1 && csk > 0) cluster_wait();
    if (csk > 0 && p.inbox_in_ring) {
      cluster_arrive_relaxed();
      cluster_wait();
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    // Eight warps: warp w may read TMEM lanes [32 * (w % 4), +32), so two warps share
    // each lane quarter and take alternate 64-column groups of the tile.  One warp per
    // scheduler is latency-bound on its own dependent instruction stream; two hide
    // each other's TMEM-load, conversion and store latencies.
    const int q = warp & 3;                          // TMEM lane quarter
    const int wsub = (warp - 2) >> 2;                // 0 / 1: which 64-column groups
    const int epi_tid = (warp - 2) * 32 + lane;      // 0..255
    const int row_in_tile = q * 32 + lane;
    const int is_bf16 = p.is_bf16;
    const int act = T::ACT ? p.act : static_cast<int>(ACT_NONE);
    uint8_t* my_store = smem_store + (warp - 2) * T::STORE_BUF_BYTES;
    uint32_t acc = 0, acc_phase = 0;
    uint32_t bias_buf = 0;
    constexpr int CHUNKS32 = T::OUT_BN / 32 > 0 ? T::OUT_BN / 32 : 1;  // 32-column chunks
    constexpr int CHUNK_COLS = T::OUT_BN < 32 ? T::OUT_BN : 32;
    constexpr int EPI_THREADS = T::EPI_WARPS * 32;
    const uint32_t acc_empty_leader =
        (CG == 2) ? map_to_cta(bar_acc_empty, pair_base) : bar_acc_empty;
#ifdef AYLA_B200_TRACE
    bool acc_seen_stamped = false;
#endif
    AYLA_TRACE_BEGIN

    // No early exit in this loop: the warps meet at named barriers, so after an abort
    // they keep walking the units together (every wait then returns at once) and the
    // results are garbage that the status word disowns.
    UnitCursor<T> cursor(p, first_unit, unit_stride, cta_rank, csk_rank);
    WorkUnit w;
    grid_dependency_wait();  // these warps read bias / gate operands and write the output
    while (cursor.next(w)) {
      const bool split_k = T::LEAN ? false : w.is_split;

      if constexpr (T::EPI == EPI_BIAS && !T::TRANS_OUT) {
        // Stage this tile's bias slice as fp32; double buffered so one barrier per
        // tile is enough.
        float* bdst = smem_bias + bias_buf * BN;
        for (int c = epi_tid; c < BN; c += EPI_THREADS) {
          const int col = w.n0 + c;
          bdst[c] = (col < p.n) ? load_elem(p.bias, col, is_bf16) : 0.0f;
        }
        named_bar_sync(1, EPI_THREADS);
      }

      AYLA_TRACE_WAIT(tr_wait, bw.wait(bar_acc_full + acc * 8, acc_phase, ST_TIMEOUT_ACC_FULL))
#ifdef AYLA_B200_TRACE
      if (stamps != nullptr && warp == 2 && lane == 0 && !acc_seen_stamped) {
        trace_stamp(stamps, 13);
        acc_seen_stamped = true;
      }
#endif
      tc_fence_after_sync();
      const uint32_t t_acc = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;

      // Rows of the tile that exist: the matrix may end inside it, and the swapped form may
      // give a tile fewer than 128 rows.
      const int row_end = T::TRANS_OUT ? min(p.m, w.m0 + p.tile_rows) : p.m;
      const bool rows_live = (w.m0 + q * 32) < row_end;
      const int unit_chunks = w.is_narrow ? CHUNKS32 / 2 : CHUNKS32;
      const int unit_groups = (unit_chunks + 1) / 2;

      // Hand the accumulator buffer back to the MMA warp (every warp arrives once per
      // unit, after its last TMEM load has completed).  The MMA warp waits for that only before
      // the unit ACC_BUFS later: the last arrivals of a CTA would find nobody waiting, and for
      // a CTA pair they would be remote arrivals still in flight when the leader leaves, so
      // they are not sent.
      static_assert(T::ACC_BUFS <= 2, "UnitCursor::follows looks at most two units ahead");
      const bool release_awaited = cursor.follows(T::ACC_BUFS);
      auto release_accumulator = [&]() {
        if (!release_awaited) return;
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if constexpr (CG == 2) {
            mbar_arrive_cluster(acc_empty_leader + acc * 8);
          } else {
            mbar_arrive(bar_acc_empty + acc * 8);
          }
        }
      };

      // Gate (activation variants, row-major output): multiply this thread's 32 values of chunk
      // `c32` by the matching elements of `mul`, which has the shape and layout of `out`.
      auto gate_chunk = [&](float (&v)[32], int c32) {
        if constexpr (T::ACT && !T::TRANS_OUT) {
          const int row = w.m0 + row_in_tile;
          const int col0 = w.n0 + c32 * 32;
          if (p.mul == nullptr || row >= p.m) return;
          if (p.mul_per_row) {
            const float g = load_elem(p.mul, w.batch * static_cast<long long>(p.m) + row, is_bf16);
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= g;
            return;
          }
          const uint8_t* src = reinterpret_cast<const uint8_t*>(p.mul) +
                               2 * (w.batch * p.out_batch_stride + static_cast<long long>(row) * p.out_ld + col0);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (col0 + 8 * j < p.n) {
              const uint4 g = *reinterpret_cast<const uint4*>(src + 16 * j);
              const float2 g0 = unpack2(g.x, is_bf16), g1 = unpack2(g.y, is_bf16);
              const float2 g2 = unpack2(g.z, is_bf16), g3 = unpack2(g.w, is_bf16);
              v[8 * j + 0] *= g0.x;
              v[8 * j + 1] *= g0.y;
              v[8 * j + 2] *= g1.x;
              v[8 * j + 3] *= g1.y;
              v[8 * j + 4] *= g2.x;
              v[8 * j + 5] *= g2.y;
              v[8 * j + 6] *= g3.x;
              v[8 * j + 7] *= g3.y;
            }
          }
        }
      };
      // The same for one element of the transposed or narrow-slice forms (`index` as into `out`,
      // `out_row` the element's row of the output matrix).
      auto gate_elem = [&](float x, long long index, int out_row) {
        if constexpr (T::ACT) {
          if (p.mul != nullptr) {
            const long long at = p.mul_per_row
                                     ? w.batch * static_cast<long long>(T::TRANS_OUT ? p.n : p.m) + out_row
                                     : w.batch * p.out_batch_stride + index;
            return x * load_elem(p.mul, at, is_bf16);
          }
        }
        return x;
      };

      // Finish one chunk of up to 32 fp32 values of this thread's row (bias, round,
      // store).  `c32` indexes 32-column chunks of the output tile.
      auto finish_chunk = [&](float (&v)[32], int c32) {
        if constexpr (T::TRANS_OUT) {
          // Kernel rows are output columns: out[batch][col][row].
          const int row = w.m0 + row_in_tile;
          float bias_v = 0.0f;
          if constexpr (T::EPI == EPI_BIAS) {
            if (row < row_end) bias_v = load_elem(p.bias, row, is_bf16);
          }
          if (row < row_end) {
            uint8_t* base = reinterpret_cast<uint8_t*>(p.out) + 2 * (w.batch * p.out_batch_stride);
            if constexpr (T::EPI == EPI_BIAS) {
#pragma unroll
              for (int j = 0; j < CHUNK_COLS; ++j) v[j] += bias_v;
            }
            apply_act_chunk<CHUNK_COLS>(v, act);
#pragma unroll
            for (int j = 0; j < CHUNK_COLS; ++j) {
              const int col = w.n0 + c32 * 32 + j;
              if (col < p.n) {
                const long long at = static_cast<long long>(col) * p.out_ld + row;
                store_elem(base, at, gate_elem(v[j], at, col), is_bf16);
              }
            }
          }
        } else {
          if constexpr (T::EPI == EPI_BIAS) {
            const float4* b4 = reinterpret_cast<const float4*>(smem_bias + bias_buf * BN + c32 * 32);
#pragma unroll
            for (int j = 0; j < CHUNK_COLS / 4; ++j) {
              const float4 b = b4[j];
              v[4 * j + 0] += b.x;
              v[4 * j + 1] += b.y;
              v[4 * j + 2] += b.z;
              v[4 * j + 3] += b.w;
            }
          }
          apply_act_chunk<CHUNK_COLS>(v, act);
          gate_chunk(v, c32);
          // Two 32-column chunks fill one 64-column (128-byte) store row.
          const int half = c32 & 1;
          if (half == 0) {
            // The bulk store this warp issued last must have finished reading the buffer.
            if (lane == 0) tma_store_wait_read<0>();
            __syncwarp();
          }
          uint32_t pk[CHUNK_COLS / 2];
          if (is_bf16) {
#pragma unroll
            for (int j = 0; j < CHUNK_COLS / 2; ++j) {
              __nv_bfloat162 t = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
              pk[j] = *reinterpret_cast<uint32_t*>(&t);
            }
          } else {
#pragma unroll
            for (int j = 0; j < CHUNK_COLS / 2; ++j) {
              __half2 t = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
              pk[j] = *reinterpret_cast<uint32_t*>(&t);
            }
          }
#pragma unroll
          for (int j = 0; j < CHUNK_COLS / 8; ++j) {
            const int chunk16 = half * 4 + j;  // 16-byte chunk within the 128-byte row
            *reinterpret_cast<uint4*>(my_store + lane * 128 + ((chunk16 ^ (lane & 7)) << 4)) =
                make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
          }
#ifdef AYLA_B200_TRACE
          if (stamps != nullptr && warp == 2 && lane == 0 && c32 < 2) trace_stamp(stamps, 22 + c32);
#endif
          if (half == 1) {
            fence_proxy_async_smem();
#ifdef AYLA_B200_TRACE
            if (stamps != nullptr && warp == 2 && lane == 0 && c32 < 2) trace_stamp(stamps, 24);
#endif
            __syncwarp();
            if (lane == 0) {
              tma_store_3d(&tm_d, smem_u32(my_store), w.n0 + (c32 >> 1) * 64, w.m0 + q * 32, w.batch);
              tma_store_commit();
            }
#ifdef AYLA_B200_TRACE
            if (stamps != nullptr && warp == 2 && lane == 0 && c32 < 2) trace_stamp(stamps, 25);
#endif
          }
        }
      };

      if (csk > 0) {
        // ---- cluster split-K: S CTAs of the cluster (those with this CTA's place in its
        // pair) hold the S partial sums of this 128-row tile.  Each owns BN / S columns of
        // it: every CTA sends each owner its partial of the owner's columns with asynchronous
        // stores into the owner's inbox (distributed shared memory), each store crediting the
        // owner's inbox barrier with its bytes; an owner waits for that barrier alone, adds
        // the S partials in split order and stores.  Nobody waits for a sender's stores but
        // their receiver.
        if constexpr (T::EPI != EPI_SWIGLU) {
          const int slice_cols = BN / csk;
          const int slice_shift = __ffs(slice_cols) - 1;
          const int slice_c4 = slice_cols >> 2;
          const uint32_t exch = smem_u32(smem) + p.inbox_offset;
          // A CTA keeps its own partial of its own columns in TMEM (no trip through shared
          // memory) whenever a 32-column TMEM load never straddles two owners.
          const bool own_in_tmem = slice_cols >= CHUNK_COLS;
          if constexpr (CG == 1) cluster_wait();  // every CTA of the cluster has its inbox barrier ready
          if (p.inbox_in_ring) {
            // Every CTA's MMAs are done (its epilogue warps have seen the accumulator): no ring
            // is being read any more.  The threads only meet here; nothing is published.
            cluster_arrive_relaxed();
            cluster_wait();
          }
#ifdef AYLA_B200_TRACE
          if (stamps != nullptr && warp == 2 && lane == 0) trace_stamp(stamps, 6);
#endif
          auto send_chunk = [&](int c32, const uint32_t (&r)[32]) {
#pragma unroll
            for (int j = 0; j < CHUNK_COLS / 4; ++j) {
              const int col = c32 * 32 + 4 * j;
              const int owner = col >> slice_shift;
              if (own_in_tmem && owner == csk_rank) continue;
              const int c4 = (col - (owner << slice_shift)) >> 2;
              const uint32_t owner_cta = static_cast<uint32_t>(owner * CG) + cta_rank;
              // An owner that keeps its own partial in TMEM has no inbox slot for itself.
              const int slot = (own_in_tmem && csk_rank > owner) ? csk_rank - 1 : csk_rank;
              const uint32_t dst =
                  map_to_cta(exch + ((slot * slice_c4 + c4) * 128 + row_in_tile) * 16, owner_cta);
              st_async_v4(dst, __uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                          __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]),
                          map_to_cta(bar_inbox, owner_cta));
            }
          };
          {
            // The chunks that hold other owners' columns, dealt alternately to the two warps
            // of a lane quarter and sent two at a time (both TMEM loads in flight together).
            const int own_c0 = own_in_tmem ? (csk_rank << slice_shift) >> 5 : -1;
            const int own_c1 = own_in_tmem ? own_c0 + (slice_cols >> 5) : -1;
            int pending = -1, seen = 0;
            uint32_t ra[32], rb[32];
#pragma unroll 1
            for (int c32 = 0; c32 < CHUNKS32; ++c32) {
              if (c32 >= own_c0 && c32 < own_c1) continue;
              const bool mine = ((seen++) & 1) == wsub;
              if (!mine) continue;
              if constexpr (CHUNK_COLS == 32) {
                if (pending < 0) {
                  tmem_ld_32x32(t_acc + c32 * 32, ra);
                  pending = c32;
                } else {
                  tmem_ld_32x32(t_acc + c32 * 32, rb);
                  tmem_ld_wait();
                  send_chunk(pending, ra);
                  send_chunk(c32, rb);
                  pending = -1;
                }
              } else {
                tmem_ld_32x16(t_acc, *reinterpret_cast<uint32_t(*)[16]>(&ra[0]));
                tmem_ld_wait();
                send_chunk(c32, ra);
              }
            }
            if (pending >= 0) {
              tmem_ld_wait();
              send_chunk(pending, ra);
            }
          }
#ifdef AYLA_B200_TRACE
          if (stamps != nullptr && warp == 2 && lane == 0) trace_stamp(stamps, 15);
#endif
          // The partials of this CTA's columns have all landed when the inbox barrier completes.
          bw.wait(bar_inbox, 0, ST_TIMEOUT_INBOX);
#ifdef AYLA_B200_TRACE
          if (stamps != nullptr && warp == 2 && lane == 0) trace_stamp(stamps, 7);
#endif
          const float4* mine = reinterpret_cast<const float4*>(smem + p.inbox_offset);
          const int row = w.m0 + row_in_tile;
          if (own_in_tmem) {
            // Sum, in split order, the partials of this CTA's columns: its own from TMEM,
            // the others from the exchange area.  `lc` counts 32-column chunks of the slice.
            // All eight loads of a peer's partial are issued before any is added (summing element
            // by element inside the loop over the splits left every load's latency exposed: 0.8 us
            // per chunk measured).
            auto reduce_chunk = [&](int lc, const uint32_t (&own)[32], float (&v)[32]) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = 0.0f;
#pragma unroll 1
              for (int s = 0; s < csk; ++s) {
                if (s == csk_rank) {
#pragma unroll
                  for (int j = 0; j < 32; ++j) v[j] += __uint_as_float(own[j]);
                } else {
                  const float4* src = mine + ((s > csk_rank ? s - 1 : s) * slice_c4 + lc * 8) * 128 + row_in_tile;
                  float4 x[8];
#pragma unroll
                  for (int j = 0; j < 8; ++j) x[j] = src[j * 128];
#pragma unroll
                  for (int j = 0; j < 8; ++j) {
                    v[4 * j + 0] += x[j].x;
                    v[4 * j + 1] += x[j].y;
                    v[4 * j + 2] += x[j].z;
                    v[4 * j + 3] += x[j].w;
                  }
                }
              }
            };
            const int first_c32 = (csk_rank << slice_shift) >> 5;  // tile chunk index of the slice
            const int slice_chunks = slice_cols >> 5;
            if constexpr (CHUNK_COLS == 32) {
#pragma unroll 1
              for (int lc = wsub; lc < slice_chunks; lc += 2) {
                const int c32 = first_c32 + lc;
                uint32_t ra[32];
                tmem_ld_32x32(t_acc + c32 * 32, ra);
                tmem_ld_wait();
#ifdef AYLA_B200_TRACE
                if (stamps != nullptr && warp == 2 && lane == 0 && lc == wsub) trace_stamp(stamps, 26);
#endif
                float v[32];
                reduce_chunk(lc, ra, v);
#ifdef AYLA_B200_TRACE
                if (stamps != nullptr && warp == 2 && lane == 0 && lc == wsub) trace_stamp(stamps, 27);
#endif
                const int col0 = w.n0 + c32 * 32;
                if (!(rows_live && col0 < p.n)) continue;
                if constexpr (T::TRANS_OUT) {
                  finish_chunk(v, c32);
                } else if (row < row_end) {
                  // A lone 32-column chunk: 64 contiguous bytes of this thread's output row.
                  if constexpr (T::EPI == EPI_BIAS) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] += smem_bias[bias_buf * BN + c32 * 32 + j];
                  }
                  apply_act_chunk<32>(v, act);
                  gate_chunk(v, c32);
                }
                // Through this warp's staging rows, so that one store instruction writes eight
                // rows of 64 contiguous bytes instead of 16 bytes of each of 32 rows (the load/store
                // unit takes a cycle per 128-byte line touched: 0.6 us for the tile the direct way).
                // Row r holds its four 16-byte pieces at r * 64, piece c at position c ^ ((r >> 1) & 3).
                if constexpr (!T::TRANS_OUT) {
                  __syncwarp();
                  if (row < row_end) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                      *reinterpret_cast<uint4*>(my_store + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4)) =
                          make_uint4(pack2(v[8 * j], v[8 * j + 1], is_bf16), pack2(v[8 * j + 2], v[8 * j + 3], is_bf16),
                                     pack2(v[8 * j + 4], v[8 * j + 5], is_bf16), pack2(v[8 * j + 6], v[8 * j + 7], is_bf16));
                    }
                  }
                  __syncwarp();
                  const int piece = lane & 3;
                  const int col = col0 + piece * 8;
                  uint8_t* dst0 = reinterpret_cast<uint8_t*>(p.out) + 2 * (w.batch * p.out_batch_stride + col);
#pragma unroll
                  for (int i = 0; i < 4; ++i) {
                    const int r = i * 8 + (lane >> 2);
                    const int out_row = w.m0 + q * 32 + r;
                    const uint4 x = *reinterpret_cast<const uint4*>(my_store + r * 64 + ((piece ^ ((r >> 1) & 3)) << 4));
                    if (out_row < row_end && col < p.n) {
                      *reinterpret_cast<uint4*>(dst0 + 2 * static_cast<long long>(out_row) * p.out_ld) = x;
                    }
                  }
                }
              }
            }
          } else if (row < row_end) {
            // Narrow slices (fewer than 32 columns per CTA): every partial, this CTA's own
            // included, went through the exchange area.
            uint8_t* base = reinterpret_cast<uint8_t*>(p.out) + 2 * (w.batch * p.out_batch_stride);
            for (int c4 = wsub; c4 < slice_c4; c4 += 2) {
              float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
              for (int s = 0; s < csk; ++s) {
                const float4 x = mine[(s * slice_c4 + c4) * 128 + row_in_tile];
                sum.x += x.x;
                sum.y += x.y;
                sum.z += x.z;
                sum.w += x.w;
              }
              const int col = w.n0 + csk_rank * slice_cols + c4 * 4;
              if (col < p.n) {
                float v4[4] = {sum.x, sum.y, sum.z, sum.w};
                if constexpr (T::TRANS_OUT) {
                  float bias_v = 0.0f;
                  if constexpr (T::EPI == EPI_BIAS) bias_v = load_elem(p.bias, row, is_bf16);
#pragma unroll
                  for (int j = 0; j < 4; ++j) v4[j] += bias_v;
                  apply_act_chunk<4>(v4, act);
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    if (col + j < p.n) {
                      const long long at = static_cast<long long>(col + j) * p.out_ld + row;
                      store_elem(base, at, gate_elem(v4[j], at, col + j), is_bf16);
                    }
                  }
                } else {
                  if constexpr (T::EPI == EPI_BIAS) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) v4[j] += load_elem(p.bias, col + j, is_bf16);
                  }
                  apply_act_chunk<4>(v4, act);
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    v4[j] = gate_elem(v4[j], static_cast<long long>(row) * p.out_ld + col + j, row);
                  }
                  uint2 pk;
                  pk.x = pack2(v4[0], v4[1], is_bf16);
                  pk.y = pack2(v4[2], v4[3], is_bf16);
                  *reinterpret_cast<uint2*>(base + 2 * (static_cast<long long>(row) * p.out_ld + col)) = pk;
                }
              }
            }
          }
          release_accumulator();
        }
      } else if (!split_k) {
        if constexpr (!T::TRANS_OUT) {
          // This warp's 64-column groups, software-pipelined over 32-column chunks: the
          // TMEM load of the next chunk is in flight while this one is converted,
          // staged and stored.
          constexpr int REGS = (T::EPI == EPI_SWIGLU) ? 64 : 32;
          uint32_t ra[REGS], rb[REGS];
          auto issue = [&](int c32, uint32_t (&r)[REGS]) {
            if constexpr (T::EPI == EPI_SWIGLU) {
              tmem_ld_32x32(t_acc + c32 * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
              tmem_ld_32x32(t_acc + T::OUT_BN + c32 * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
            } else {
              tmem_ld_32x32(t_acc + c32 * 32, r);
            }
          };
          auto consume = [&](int c32, uint32_t (&r)[REGS]) {
            // Liveness per 64 columns: both halves of a 128-byte store row go together.
            if (!(rows_live && (w.n0 + (c32 >> 1) * 64) < p.n)) return;
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if constexpr (T::EPI == EPI_SWIGLU) {
                v[j] = silu_mul(__uint_as_float(r[j]), __uint_as_float(r[32 + j]));
              } else {
                v[j] = __uint_as_float(r[j]);
              }
            }
            finish_chunk(v, c32);
          };
          if (wsub >= unit_groups) {
            release_accumulator();
          } else {
            issue(2 * wsub, ra);
#pragma unroll 1
            for (int g = wsub; g < unit_groups; g += 2) {
              tmem_ld_wait();
#ifdef AYLA_B200_TRACE
              if (stamps != nullptr && warp == 2 && lane == 0 && g == wsub) trace_stamp(stamps, 16);
#endif
              issue(2 * g + 1, rb);
              consume(2 * g, ra);
              tmem_ld_wait();
              if (g + 2 < unit_groups) {
                issue(2 * (g + 2), ra);
              } else {
                release_accumulator();
              }
              consume(2 * g + 1, rb);
#ifdef AYLA_B200_TRACE
              if (stamps != nullptr && warp == 2 && lane == 0 && (g >> 1) < 4) trace_stamp(stamps, 18 + (g >> 1));
#endif
            }
          }
        } else {
          // Transposed form: chunks alternate between the two warps of a lane quarter.
#pragma unroll 1
          for (int c32 = wsub; c32 < CHUNKS32; c32 += 2) {
            const bool live = rows_live && (w.n0 + c32 * 32) < p.n;
            float v[32];
            if constexpr (CHUNK_COLS == 32) {
              uint32_t r[32];
              tmem_ld_32x32(t_acc + c32 * 32, r);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
            } else {
              uint32_t r[16];
              tmem_ld_32x16(t_acc, r);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
            }
            if (c32 + 2 >= CHUNKS32) release_accumulator();
            if (live) finish_chunk(v, c32);
          }
          if (wsub >= CHUNKS32) release_accumulator();
        }
      } else {
        // ---- split-K: park the fp32 partial, last arriver of the tile reduces.
        // Slab layout: float4 index (c4, row) -> c4 * 128 + row, so a warp's
        // 16-byte accesses are contiguous.  64-column groups (32-column chunks in the
        // transposed form) alternate between the two warps of a lane quarter.
        if constexpr (T::EPI != EPI_SWIGLU) {
          constexpr int STEP = T::TRANS_OUT ? 1 : 2;  // chunks handled back to back
          float4* slab = reinterpret_cast<float4*>(p.ws) +
                         static_cast<size_t>(cursor.slab_of(w, w.split)) * (32 * BN);
#pragma unroll 1
          for (int c0 = wsub * STEP; c0 < CHUNKS32; c0 += 2 * STEP) {
#pragma unroll 1
            for (int c32 = c0; c32 < c0 + STEP && c32 < CHUNKS32; ++c32) {
              if constexpr (CHUNK_COLS == 32) {
                uint32_t r[32];
                tmem_ld_32x32(t_acc + c32 * 32, r);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  slab[(c32 * 8 + j) * 128 + row_in_tile] =
                      make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                  __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                }
              } else {
                uint32_t r[16];
                tmem_ld_32x16(t_acc, r);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  slab[j * 128 + row_in_tile] =
                      make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                  __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                }
              }
            }
          }
          release_accumulator();
          __threadfence();
          named_bar_sync(2, EPI_THREADS);
          if (epi_tid == 0) {
            const unsigned old = atomicAdd(p.counters + w.counter, 1u);
            const bool last = (old == static_cast<unsigned>(w.nsplit - 1));
            if (last) p.counters[w.counter] = 0;  // leave the counter clean for the next launch
            *last_flag = last ? 1u : 0u;
          }
          named_bar_sync(2, EPI_THREADS);
          const bool last = *last_flag != 0;
          if (last) {
            __threadfence();
            const float4* all_slabs = reinterpret_cast<const float4*>(p.ws);
#pragma unroll 1
            for (int c0 = wsub * STEP; c0 < CHUNKS32; c0 += 2 * STEP) {
#pragma unroll 1
              for (int c32 = c0; c32 < c0 + STEP && c32 < CHUNKS32; ++c32) {
                float v[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = 0.0f;
                // Two partials per round trip (both loads issued before either is summed);
                // the order of the additions is still split 0, 1, 2, ...
                for (int s = 0; s < w.nsplit; s += 2) {
                  const bool two = s + 1 < w.nsplit;
                  const float4* sl0 = all_slabs + static_cast<size_t>(cursor.slab_of(w, s)) * (32 * BN);
                  const float4* sl1 =
                      two ? all_slabs + static_cast<size_t>(cursor.slab_of(w, s + 1)) * (32 * BN) : sl0;
                  float4 x0[CHUNK_COLS / 4], x1[CHUNK_COLS / 4];
#pragma unroll
                  for (int j = 0; j < CHUNK_COLS / 4; ++j) x0[j] = __ldcg(sl0 + (c32 * 8 + j) * 128 + row_in_tile);
#pragma unroll
                  for (int j = 0; j < CHUNK_COLS / 4; ++j) x1[j] = __ldcg(sl1 + (c32 * 8 + j) * 128 + row_in_tile);
#pragma unroll
                  for (int j = 0; j < CHUNK_COLS / 4; ++j) {
                    v[4 * j + 0] += x0[j].x;
                    v[4 * j + 1] += x0[j].y;
                    v[4 * j + 2] += x0[j].z;
                    v[4 * j + 3] += x0[j].w;
                  }
                  if (two) {
#pragma unroll
                    for (int j = 0; j < CHUNK_COLS / 4; ++j) {
                      v[4 * j + 0] += x1[j].x;
                      v[4 * j + 1] += x1[j].y;
                      v[4 * j + 2] += x1[j].z;
                      v[4 * j + 3] += x1[j].w;
                    }
                  }
                }
                const bool live = rows_live && (w.n0 + c32 * 32) < p.n;
                const bool live64 = rows_live && (w.n0 + (c32 >> 1) * 64) < p.n;
                if (T::TRANS_OUT ? live : live64) finish_chunk(v, c32);
              }
            }
          }
          // Every warp must have read last_flag before the next unit rewrites it.
          named_bar_sync(2, EPI_THREADS);
        }
      }

      if constexpr (T::EPI == EPI_BIAS && !T::TRANS_OUT) bias_buf ^= 1;
      if (++acc == T::ACC_BUFS) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
#ifdef AYLA_B200_TRACE
    if (stamps != nullptr && warp == 2 && lane == 0) trace_stamp(stamps, 17);
#endif
    if constexpr (!T::TRANS_OUT) {
      // Shared memory must outlive the bulk stores that read it; their global writes are
      // complete, like every other store of the grid, when the grid is.
      if (lane == 0) tma_store_wait_read<0>();
    }
    if (warp == 2) {
      AYLA_TRACE_END(2)
#ifdef AYLA_B200_TRACE
      if (stamps != nullptr && lane == 0) trace_stamp(stamps, 4);
#endif
    }
  }

  // ------------------------------------------------------------------ teardown
  if (bw.aborted()) {
    // Give copies and MMAs that are still in flight time to land before shared
    // memory and TMEM are released.
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (CG == 2) {
    // The leader's MMAs write the peer's TMEM and both CTAs' barriers: neither
    // CTA may free TMEM or exit before both are done.  Nothing is published by this meeting:
    // every remote arrival a thread of either CTA sent has been waited for by its receiver, and
    // the arrivals of the leader's commits on the peer's slot barriers precede the one on its
    // accumulator barrier, which the peer's epilogue warps have seen.
    cluster_arrive_relaxed();
    cluster_wait();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<CG>(tmem_base, T::TMEM_COLS);
  }
#ifdef AYLA_B200_TRACE
  if (stamps != nullptr && threadIdx.x == 32) {
    trace_stamp(stamps, 5);
    long long* out = p.trace + 4096 + blockIdx.x * 64;
    for (int i = 0; i < 40; ++i) out[i] = stamps[i];
  }
#endif
#endif
}

}  // namespace ayla_b200
