// C ABI of the sm_100a GEMM backend: argument checks, schedule choice, tensor-map
// encoding and the kernel launch.  Nothing here allocates device memory or
// synchronises, so every entry point except ayla_b200_init can run inside CUDA
// graph capture.
#include "../../include/ayla_b200.h"

#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>

#include "kernel_registry.h"

namespace ayla_b200 {
namespace {

thread_local std::string g_last_error;

int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return code;
}

constexpr int kMaxVariants = 128;
constexpr int kMaxDevices = 64;

struct Registry {
  KernelEntry entries[kMaxVariants];
  int count = 0;
  Registry() {
    append_variants_cg1(entries, &count);
    append_variants_cg2(entries, &count);
    append_variants_trans(entries, &count);
    append_variants_swiglu(entries, &count);
    base_count = count;
    append_variants_act_cg1(entries, &count);
    append_variants_act_cg2(entries, &count);
    append_variants_act_trans(entries, &count);
    append_variants_lean_cg1(entries, &count);
    append_variants_lean_cg2(entries, &count);
    append_variants_lean_trans(entries, &count);
    append_variants_lean_act_cg1(entries, &count);
    append_variants_lean_act_cg2(entries, &count);
    append_variants_lean_act_trans(entries, &count);
  }
  int base_count = 0;  // the variants without the activation epilogue come first
  // `lean` asks for the variant without the k-split epilogues; where there is none the full
  // variant serves.
  const KernelEntry* find(int tile_n, int cta_group, int epilogue, int transposed, int activation = 0,
                          int lean = 0) const {
    const KernelEntry* full = nullptr;
    for (int i = 0; i < count; ++i) {
      const KernelEntry& e = entries[i];
      if (e.tile_n == tile_n && e.cta_group == cta_group && e.epilogue == epilogue &&
          e.transposed_out == transposed && e.activation == activation) {
        if (e.lean == lean) return &e;
        if (e.lean == 0) full = &e;
      }
    }
    return full;
  }
};

const Registry& registry() {
  static const Registry r;
  return r;
}

struct DeviceState {
  std::atomic<bool> ready{false};
  int sm_count = 0;
};
DeviceState g_devices[kMaxDevices];
std::mutex g_init_mutex;
PFN_cuTensorMapEncodeTiled g_encode_tiled = nullptr;
std::atomic<long long> g_timeout_ns{2000000000ll};
std::atomic<int> g_debug_flags{0};
std::atomic<int> g_launch_overlap{1};

// ------------------------------------------------------------- tensor maps

struct MapKey {
  const void* ptr;
  uint64_t d0, d1, d2;
  uint32_t b0, b1, b2;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && d0 == o.d0 && d1 == o.d1 && d2 == o.d2 && b0 == o.b0 && b1 == o.b1 &&
           b2 == o.b2;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = reinterpret_cast<uint64_t>(k.ptr) * 0x9E3779B97F4A7C15ull;
    h ^= (k.d0 + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
    h ^= (k.d1 + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
    h ^= (k.d2 + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
    h ^= ((static_cast<uint64_t>(k.b0) << 40) ^ (static_cast<uint64_t>(k.b1) << 20) ^ k.b2) +
         (h << 6) + (h >> 2);
    return static_cast<size_t>(h);
  }
};

// Descriptors are pure functions of (pointer, extents, box); cache them by value
// as the reference's launcher does (ayla/ptx_runtime.py:185-235), behind a mutex
// because this library does not rely on the GIL.
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_map_cache;
std::mutex g_map_mutex;

// 3-D map over a row-major [d2][d1][d0] tensor of 16-bit elements, box
// [b2][b1][b0], 128-byte swizzle (b0 must be 64 elements).
int encode_map(CUtensorMap* out, const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint32_t b0,
               uint32_t b1, uint32_t b2) {
  const MapKey key{ptr, d0, d1, d2, b0, b1, b2};
  {
    std::lock_guard<std::mutex> lock(g_map_mutex);
    auto it = g_map_cache.find(key);
    if (it != g_map_cache.end()) {
      *out = it->second;
      return AYLA_B200_OK;
    }
  }
  const cuuint64_t dims[3] = {d0, d1, d2};
  const cuuint64_t strides[2] = {d0 * 2, d0 * d1 * 2};
  const cuuint32_t box[3] = {b0, b1, b2};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  const CUresult r = g_encode_tiled(
      out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box,
      elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    return fail(AYLA_B200_E_CUDA,
                "cuTensorMapEncodeTiled failed (%d) for ptr=%p dims=[%llu,%llu,%llu] box=[%u,%u,%u]",
                static_cast<int>(r), ptr, (unsigned long long)d0, (unsigned long long)d1,
                (unsigned long long)d2, b0, b1, b2);
  }
  std::lock_guard<std::mutex> lock(g_map_mutex);
  if (g_map_cache.size() > 8192) g_map_cache.clear();
  g_map_cache.emplace(key, *out);
  return AYLA_B200_OK;
}

// ------------------------------------------------------------ the schedule

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// The problem as the kernel sees it after an optional swap of the operands.
struct Problem {
  int64_t rows, cols, k, batch;  // rows fill the 128-row tile, cols the accumulator width
  const void* row_operand;       // [batch][rows][k]
  const void* col_operand;       // [batch][cols][k]
};

struct Plan {
  const KernelEntry* kernel;
  int m_tiles, n_tiles, k_blocks, splits, kb_per_split, total_units, group_m, grid;
  int split_from_tile;  // first k-split tile (0 = all tiles split, == tiles when none is)
  int narrow_from_tile; // first tile done as two half-width units (== tiles when none is)
  int stream_k, kb_per_cta;
  int cluster_split;    // cluster size of the cluster split-K schedule (0 = not used)
  long long slabs;      // fp32 partial-sum slabs of 128 x tile_n the schedule may write
  int row_tiles;  // 128-row x tile_n tiles (split-K counters, slabs)
  int tile_rows;  // rows of the row operand per tile (128 unless the swapped form trims it)
};

int check_shape(int op, int dtype, int64_t batch, int64_t m, int64_t n, int64_t k) {
  if (op != AYLA_B200_OP_MM && op != AYLA_B200_OP_ADDMM && op != AYLA_B200_OP_BMM) {
    return fail(AYLA_B200_E_INVALID, "unknown op %d", op);
  }
  if (dtype != AYLA_B200_F16 && dtype != AYLA_B200_BF16) {
    return fail(AYLA_B200_E_INVALID, "unknown dtype %d (0 = float16, 1 = bfloat16)", dtype);
  }
  if (batch <= 0 || m <= 0 || n <= 0 || k <= 0) {
    return fail(AYLA_B200_E_INVALID, "non-positive extent batch=%lld m=%lld n=%lld k=%lld",
                (long long)batch, (long long)m, (long long)n, (long long)k);
  }
  if (op != AYLA_B200_OP_BMM && batch != 1) {
    return fail(AYLA_B200_E_INVALID, "batch must be 1 for mm/addmm, got %lld", (long long)batch);
  }
  if (n % 8 != 0) {
    return fail(AYLA_B200_E_UNSUPPORTED, "n=%lld must be a multiple of 8 (16-byte output rows)",
                (long long)n);
  }
  if (k % 8 != 0) {
    return fail(AYLA_B200_E_UNSUPPORTED, "k=%lld must be a multiple of 8 (16-byte operand rows)",
                (long long)k);
  }
  if (m > 0x7FFFFFFF / 2 || n > 0x7FFFFFFF / 2 || k > 0x7FFFFFFF / 2 || batch > 65535 * 16) {
    return fail(AYLA_B200_E_UNSUPPORTED, "extent too large for 32-bit tile coordinates");
  }
  return AYLA_B200_OK;
}

int check_config(const ayla_b200_config& c, bool swiglu) {
  if (c.cta_group != 1 && c.cta_group != 2) {
    return fail(AYLA_B200_E_UNSUPPORTED, "cta_group must be 1 or 2, got %d", c.cta_group);
  }
  if (c.split_k < 1 || c.group_m < 1 || c.grid_ctas < 0) {
    return fail(AYLA_B200_E_UNSUPPORTED, "split_k and group_m must be >= 1, grid_ctas >= 0");
  }
  if (c.split_tail < 0 || c.split_tail > 2) {
    return fail(AYLA_B200_E_UNSUPPORTED, "split_tail must be 0, 1 or 2");
  }
  if (c.cluster_split != 0 && c.cluster_split != 1) {
    return fail(AYLA_B200_E_UNSUPPORTED, "cluster_split must be 0 or 1");
  }
  if (c.cluster_split) {
    if (swiglu || c.stream_k || c.split_tail) {
      return fail(AYLA_B200_E_UNSUPPORTED,
                  "cluster_split excludes stream_k, split_tail and the SwiGLU kernel");
    }
    // The cluster has split_k * cta_group CTAs, 8 at most.
    if (c.split_k != 2 && c.split_k != 4 && !(c.split_k == 8 && c.cta_group == 1)) {
      return fail(AYLA_B200_E_UNSUPPORTED,
                  "cluster_split needs split_k in {2, 4, 8} and a cluster (split_k * cta_group) of at most 8 CTAs");
    }
    if (c.tile_n % (4 * c.split_k) != 0 || (c.tile_n & (c.tile_n - 1)) != 0) {
      return fail(AYLA_B200_E_UNSUPPORTED,
                  "cluster_split needs a power-of-two tile_n that is a multiple of 4 * split_k");
    }
  }
  if (c.l2_prefetch < 0 || c.l2_prefetch > 256) {
    return fail(AYLA_B200_E_UNSUPPORTED, "l2_prefetch must be between 0 and 256 k-blocks");
  }
  if (c.early_prefetch < 0 || c.early_prefetch > 32) {
    return fail(AYLA_B200_E_UNSUPPORTED, "early_prefetch must be between 0 and 32 k-blocks");
  }
  if (c.stream_k != 0 && c.stream_k != 1) {
    return fail(AYLA_B200_E_UNSUPPORTED, "stream_k must be 0 or 1");
  }
  if (c.stream_k && (swiglu || c.split_k != 1 || c.split_tail != 0)) {
    return fail(AYLA_B200_E_UNSUPPORTED, "stream_k excludes split_k > 1, split_tail and the SwiGLU kernel");
  }
  if (c.split_tail == 2 && (swiglu || c.swap_ab || c.split_k != 1 || c.tile_n % 128 != 0)) {
    return fail(AYLA_B200_E_UNSUPPORTED,
                "split_tail = 2 (half-width last wave) needs tile_n of 128 or 256, split_k = 1 and no swap_ab");
  }
  if (c.l2_hint_a < 0 || c.l2_hint_a > 2 || c.l2_hint_b < 0 || c.l2_hint_b > 2) {
    return fail(AYLA_B200_E_UNSUPPORTED, "L2 hints must be 0, 1 or 2");
  }
  if (swiglu) {
    if (c.split_k != 1 || c.swap_ab != 0) {
      return fail(AYLA_B200_E_UNSUPPORTED, "the SwiGLU kernel has no split-K or swapped form");
    }
    return AYLA_B200_OK;
  }
  if (c.tile_rows != 0 && (!c.swap_ab || c.tile_rows < 8 || c.tile_rows > 128)) {
    return fail(AYLA_B200_E_UNSUPPORTED, "tile_rows needs swap_ab = 1 and a value between 8 and 128 (0 = 128)");
  }
  if (c.swap_ab) {
    if (c.cta_group != 1) {
      return fail(AYLA_B200_E_UNSUPPORTED, "swap_ab is only built with cta_group == 1");
    }
    if (c.tile_n != 16 && c.tile_n != 32 && c.tile_n != 64 && c.tile_n != 128) {
      return fail(AYLA_B200_E_UNSUPPORTED, "swap_ab needs tile_n in {16,32,64,128}, got %d", c.tile_n);
    }
  } else if (c.tile_n != 64 && c.tile_n != 128 && c.tile_n != 192 && c.tile_n != 256) {
    return fail(AYLA_B200_E_UNSUPPORTED, "tile_n must be 64, 128, 192 or 256, got %d", c.tile_n);
  }
  return AYLA_B200_OK;
}

// The arrival counters live in a header of fixed size at the start of the
// workspace, whatever the shape, so one zero-initialised workspace can serve
// launches of different shapes: data slabs never overlay a counter.
constexpr int kMaxSplitKTiles = 16384;
constexpr size_t kCounterBytes = static_cast<size_t>(kMaxSplitKTiles) * 4;

// Fills `plan` for a validated config.  `epilogue` is one of EPI_*.
int make_plan(const ayla_b200_config& c, int epilogue, int64_t batch, int64_t rows, int64_t cols,
              int64_t k, int sm_count, Plan* plan, int activation = 0) {
  const int transposed = c.swap_ab ? 1 : 0;
  const int tile_n = (epilogue == EPI_SWIGLU) ? 256 : c.tile_n;
  const int lean = (c.split_k <= 1 && c.stream_k == 0) ? 1 : 0;
  const KernelEntry* e = registry().find(tile_n, c.cta_group, epilogue, transposed, activation != 0 ? 1 : 0, lean);
  if (e == nullptr) {
    return fail(AYLA_B200_E_UNSUPPORTED, "no kernel variant tile_n=%d cta_group=%d epilogue=%d swap=%d",
                tile_n, c.cta_group, epilogue, transposed);
  }
  const int out_tile_n = (epilogue == EPI_SWIGLU) ? 128 : tile_n;
  plan->kernel = e;
  plan->tile_rows = (c.swap_ab && c.tile_rows > 0) ? c.tile_rows : 128;
  plan->m_tiles = static_cast<int>(ceil_div(rows, c.swap_ab ? plan->tile_rows : 128 * c.cta_group));
  plan->n_tiles = static_cast<int>(ceil_div(cols, out_tile_n));
  plan->k_blocks = static_cast<int>(ceil_div(k, 64));
  int splits = c.split_k;
  if (splits > plan->k_blocks) splits = plan->k_blocks;
  plan->kb_per_split = static_cast<int>(ceil_div(plan->k_blocks, splits));
  plan->splits = static_cast<int>(ceil_div(plan->k_blocks, plan->kb_per_split));
  const int64_t tiles = static_cast<int64_t>(batch) * plan->m_tiles * plan->n_tiles;
  if (tiles * c.cta_group > 0x7FFFFFFF) {
    return fail(AYLA_B200_E_UNSUPPORTED, "too many tiles (%lld)", (long long)tiles);
  }
  int grid = (c.grid_ctas > 0) ? c.grid_ctas : sm_count;
  if (c.cta_group == 2) {
    grid &= ~1;
    if (grid < 2) grid = 2;
  } else if (grid < 1) {
    grid = 1;
  }
  plan->stream_k = 0;
  plan->kb_per_cta = 0;
  plan->cluster_split = 0;  // also for the stream-K plan below, which returns before the cluster branch
  if (c.stream_k) {
    // Equal contiguous shares of the (tile, k-block) sequence; a share is never shorter
    // than four k-blocks so that a segment is worth its epilogue.
    const int64_t total_kb = tiles * plan->k_blocks;
    if (total_kb > 0x7FFFFFFF) {
      return fail(AYLA_B200_E_UNSUPPORTED, "too much work for the stream-K schedule (%lld k-blocks)",
                  (long long)total_kb);
    }
    int64_t ctas = grid / c.cta_group;
    int64_t share = ceil_div(total_kb, ctas);
    const int64_t min_share = plan->k_blocks < 4 ? plan->k_blocks : 4;
    if (share < min_share) share = min_share;
    ctas = ceil_div(total_kb, share);
    if (ctas * c.cta_group > kMaxSplitKTiles) {
      return fail(AYLA_B200_E_UNSUPPORTED, "stream_k over %lld CTAs (limit %d arrival counters)",
                  (long long)(ctas * c.cta_group), kMaxSplitKTiles);
    }
    plan->stream_k = 1;
    plan->kb_per_cta = static_cast<int>(share);
    plan->splits = 1;
    plan->kb_per_split = plan->k_blocks;
    plan->split_from_tile = static_cast<int>(tiles);
    plan->narrow_from_tile = 0x7FFFFFFF;
    plan->total_units = static_cast<int>(total_kb);
    plan->row_tiles = static_cast<int>(ctas * c.cta_group);
    // No tile is cut when every share is a whole number of tiles.
    plan->slabs = (share % plan->k_blocks == 0) ? 0 : 2 * ctas * c.cta_group;
    plan->group_m = c.group_m;
    plan->grid = static_cast<int>(ctas * c.cta_group);
    return AYLA_B200_OK;
  }
  plan->cluster_split = 0;
  if (c.cluster_split) {
    // One cluster of split_k CTAs (CTA pairs) per tile, one tile per cluster; every k-split
    // must be non-empty.
    const int s_k = c.split_k;
    const int per = static_cast<int>(ceil_div(plan->k_blocks, s_k));
    if (static_cast<int64_t>(s_k - 1) * per >= plan->k_blocks) {
      return fail(AYLA_B200_E_UNSUPPORTED, "cluster_split: %d k-blocks cannot be shared by %d CTAs",
                  plan->k_blocks, s_k);
    }
    if (tiles * s_k * c.cta_group > 0x7FFFFFFF) {
      return fail(AYLA_B200_E_UNSUPPORTED, "too many tiles (%lld)", (long long)tiles);
    }
    plan->cluster_split = s_k;
    plan->splits = s_k;
    plan->kb_per_split = per;
    plan->split_from_tile = 0;
    plan->narrow_from_tile = 0x7FFFFFFF;
    plan->total_units = static_cast<int>(tiles);
    plan->row_tiles = 0;
    plan->slabs = 0;
    plan->group_m = c.group_m;
    plan->grid = static_cast<int>(tiles * s_k * c.cta_group);
    return AYLA_B200_OK;
  }
  // Tiles processed at the same time by the persistent grid.
  const int64_t wave = grid / c.cta_group;
  int64_t split_from = 0;
  if (plan->splits <= 1) {
    split_from = tiles;
  } else if (c.split_tail) {
    // Only the tiles of the last, partial wave are k-split; with less than one wave of
    // tiles that is all of them, with a whole number of waves none.
    split_from = (tiles / wave) * wave;
    if (split_from == tiles) {
      plan->splits = 1;
      plan->kb_per_split = plan->k_blocks;
    }
  }
  plan->split_from_tile = static_cast<int>(split_from);
  int64_t narrow_from = tiles;
  if (c.split_tail == 2 && tiles > wave && tiles % wave != 0) {
    // The tiles of the last, partial wave are done as two half-width units each.
    narrow_from = (tiles / wave) * wave;
  }
  // INT_MAX = no narrow units (unit indices of k-split tiles run past `tiles`).
  plan->narrow_from_tile = (narrow_from == tiles) ? 0x7FFFFFFF : static_cast<int>(narrow_from);
  const int64_t units = split_from + (tiles - split_from) * plan->splits + (tiles - narrow_from);
  if (units > 0x7FFFFFFF) {
    return fail(AYLA_B200_E_UNSUPPORTED, "too many work units (%lld)", (long long)units);
  }
  plan->total_units = static_cast<int>(units);
  plan->row_tiles = static_cast<int>((tiles - split_from) * c.cta_group);
  if (plan->splits > 1 && plan->row_tiles > kMaxSplitKTiles) {
    return fail(AYLA_B200_E_UNSUPPORTED, "split_k with %d output tiles (limit %d); use split_k = 1",
                plan->row_tiles, kMaxSplitKTiles);
  }
  plan->slabs = (plan->splits > 1) ? static_cast<long long>(plan->row_tiles) * plan->splits : 0;
  plan->group_m = c.group_m;
  if (wave > units) grid = static_cast<int>(units * c.cta_group);
  plan->grid = grid;
  return AYLA_B200_OK;
}

size_t counter_bytes_for(const Plan& p) {
  if (p.slabs <= 0) return 0;
  return kCounterBytes;
}

size_t workspace_bytes_for(const Plan& p) {
  if (p.slabs <= 0) return 0;
  return counter_bytes_for(p) + static_cast<size_t>(p.slabs) * 128 * p.kernel->tile_n * sizeof(float);
}

uint32_t make_idesc(int is_bf16, int mma_m, int mma_n) {
  // tcgen05 .kind::f16 instruction descriptor: fp32 accumulator (bits 4-5 = 1),
  // A/B element format (bits 7-9 / 10-12: 0 = f16, 1 = bf16), both operands
  // K-major (bits 15, 16 = 0), N >> 3 in bits 17-22, M >> 4 in bits 24-28.
  uint32_t d = 0;
  d |= 1u << 4;
  d |= static_cast<uint32_t>(is_bf16 ? 1 : 0) << 7;
  d |= static_cast<uint32_t>(is_bf16 ? 1 : 0) << 10;
  d |= static_cast<uint32_t>(mma_n >> 3) << 17;
  d |= static_cast<uint32_t>(mma_m >> 4) << 24;
  return d;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int current_device_state(DeviceState** out, int* device) {
  int dev = -1;
  const cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) {
    return fail(AYLA_B200_E_CUDA, "cudaGetDevice: %s", cudaGetErrorString(err));
  }
  if (dev < 0 || dev >= kMaxDevices || !g_devices[dev].ready.load(std::memory_order_acquire)) {
    return fail(AYLA_B200_E_NOT_INIT, "ayla_b200_init(%d) has not been called", dev);
  }
  *out = &g_devices[dev];
  *device = dev;
  return AYLA_B200_OK;
}

void default_config(int64_t batch, int64_t m, int64_t n, int64_t k, int sm_count,
                    ayla_b200_config* c) {
  memset(c, 0, sizeof(*c));
  c->cta_group = 1;
  c->split_k = 1;
  c->group_m = 8;
  // L2 eviction hints: `a` (re-read by every column tile) is kept, `bt` (streamed) goes first.
  // In the sweep almost any hint beat none (2-10 % on mid-size shapes); this pair won most often.
  c->l2_hint_a = 2;
  c->l2_hint_b = 1;
  const int64_t k_blocks = ceil_div(k, 64);
  if (m <= 64 && n >= 128) {
    // Weight-streaming regime: put bt's rows on the 128-row tile and M on the
    // narrow accumulator, then split K until every SM has a share of the stream.
    c->swap_ab = 1;
    c->tile_n = m <= 16 ? 16 : (m <= 32 ? 32 : 64);
    const int64_t tiles = batch * ceil_div(n, 128);
    // Split K across a cluster of 4 or 2 (summed through distributed shared memory) while
    // the whole grid still runs in one wave and every CTA keeps at least four k-blocks.
    // (Clusters of 8 measured about twice as slow as clusters of 4 on these shapes.)
    for (int s = 4; s >= 2; s /= 2) {
      if (tiles * s <= static_cast<int64_t>(sm_count) && k_blocks >= 4 * s && c->tile_n % (4 * s) == 0) {
        c->split_k = s;
        c->cluster_split = 1;
        break;
      }
    }
    c->group_m = 1;
    // Weight streaming is what early_prefetch is for: half of the CTA's share of K, 16 k-blocks at most.
    {
      const int64_t share = k_blocks / c->split_k / 2;
      c->early_prefetch = static_cast<int>(share < 16 ? share : 16);
    }
    if (c->split_k == 1 && m > 16) {
      // No room to split K (bt alone fills the SMs): with a few dozen rows of `a` the plain
      // row-major 128-wide tile, its `a` box trimmed to the rows that exist, measures 1.2-1.3x
      // faster than the swapped form (M = 32, 64 at N = 14336).
      c->swap_ab = 0;
      c->tile_n = (batch * ceil_div(n, 128) <= static_cast<int64_t>(sm_count)) ? 128 : 256;  // one wave if it fits
      c->group_m = 8;
      c->split_tail = 2;
    }
    return;
  }
  // Row-major form: pick (tile width, CTA pairing, k-split) by a small cost model fitted to
  // the B200 sweep.  Costs are in units of "one 64-deep k-block of a paired 256-wide tile at
  // full tensor rate" (about 0.28 us): a tile costs its width over the measured efficiency of
  // its shape, waves are whole, a k-split pays a fixed fix-up and every launch a fixed
  // prologue/epilogue that grows with the tile width.
  struct Shape { int tile_n, cta_group; double eff; };
  static const Shape kShapes[6] = {{256, 2, 1.00}, {256, 1, 0.88}, {128, 2, 0.80},
                                   {128, 1, 0.62}, {64, 2, 0.50}, {64, 1, 0.40}};
  double best_cost = 1e300;
  for (const Shape& sh : kShapes) {
    if (sh.cta_group == 2 && (m <= 128 || k_blocks <= 4)) continue;  // shallow K: pairing only adds set-up
    if (sh.tile_n > 64 && n * 2 <= sh.tile_n) continue;
    const int64_t ctas = sm_count / sh.cta_group;
    const int64_t tiles = batch * ceil_div(m, 128 * sh.cta_group) * ceil_div(n, sh.tile_n);
    const double tile_cost = (sh.tile_n / 256.0) / sh.eff * static_cast<double>(k_blocks);
    const double launch_cost = 6.0 + sh.tile_n / 64.0;
    for (int split = 1; split <= 16; split *= 2) {
      if (split > 1 && (k_blocks < 8 * split || tiles * split > ctas)) break;
      const int64_t units = tiles * split;
      double waves = static_cast<double>(ceil_div(units, ctas));
      int tail = 0;
      if (split == 1 && units > ctas && sh.tile_n >= 128) {
        const int64_t rest = units % ctas;
        if (rest != 0 && rest * 2 <= ctas) {
          waves -= 0.45;  // the thin last wave runs at half width
          tail = 2;
        }
      }
      // Up to four CTAs (two pairs) split K across a cluster (cheap exchange through
      // distributed shared memory); deeper splits go through the workspace, where the last
      // arriver sums `split` partial tiles one after the other.
      const bool cluster = split > 1 && split * sh.cta_group <= 4;
      // Cluster exchange: two cluster barriers plus the partial columns each CTA sends,
      // 128 x tile_n x 4 bytes x (split - 1) / split, at about 16 KB per cost unit.
      const double exchange_kb = 0.5 * sh.tile_n * (split - 1) / split;
      const double fixup = split == 1 ? 0.0 : (cluster ? 2.5 + exchange_kb / 16.0
                                                       : 4.0 + 0.9 * split * (sh.tile_n / 64.0));
      const double cost = waves * tile_cost / split + fixup + launch_cost;
      if (cost < best_cost) {
        best_cost = cost;
        c->tile_n = sh.tile_n;
        c->cta_group = sh.cta_group;
        c->split_k = split;
        c->split_tail = tail;
        c->cluster_split = cluster ? 1 : 0;
      }
    }
  }
  // bt is streamed (evict-first) only while every row tile that needs a column tile's slab runs
  // in the same raster group; with more row tiles than that it is read again later and is kept.
  if (ceil_div(m, 128 * c->cta_group) > c->group_m) c->l2_hint_b = 2;
}

int launch_plan(const Plan& plan, const ayla_b200_config& c, const Problem& pr, int is_bf16,
                const void* bias, const void* b2_operand, void* out, int64_t out_rows,
                int64_t out_cols, void* workspace, size_t workspace_bytes, uint32_t* status,
                cudaStream_t stream, int activation = 0, const void* mul = nullptr, int mul_per_row = 0) {
  const KernelEntry& e = *plan.kernel;
  LaunchArgs la;
  memset(&la, 0, sizeof(la));
  int b_box_rows = (e.epilogue == EPI_SWIGLU) ? 128 : e.tile_n / e.cta_group;
  int b_stage_rows = e.tile_n / e.cta_group;  // rows of the column operand one CTA receives per stage
  int a_box_rows = plan.tile_rows;
  // An operand that fits in a single tile is loaded with a box of just its own rows (rounded
  // up to the 8-row swizzle atom): rows of the box that lie outside the tensor are zero-filled
  // by TMA at a cost comparable to real rows, and a GEMM with a handful of rows would spend
  // most of its load time on them.  The shared-memory rows the smaller box leaves untouched
  // feed only accumulator rows / columns that are never stored.
  if (e.cta_group == 1) {
    const int rows8 = static_cast<int>(ceil_div(pr.rows, 8) * 8);
    const int cols8 = static_cast<int>(ceil_div(pr.cols, 8) * 8);
    if (plan.m_tiles == 1 && rows8 < a_box_rows) a_box_rows = rows8;
    if (plan.n_tiles == 1 && e.epilogue != EPI_SWIGLU && plan.narrow_from_tile == 0x7FFFFFFF && cols8 < b_box_rows) {
      b_box_rows = cols8;
      b_stage_rows = cols8;
    }
  }
  int rc = encode_map(&la.tm_a, pr.row_operand, pr.k, pr.rows, pr.batch, 64, a_box_rows, 1);
  if (rc) return rc;
  rc = encode_map(&la.tm_b, pr.col_operand, pr.k, pr.cols, pr.batch, 64, b_box_rows, 1);
  if (rc) return rc;
  if (e.epilogue == EPI_SWIGLU) {
    rc = encode_map(&la.tm_b2, b2_operand, pr.k, pr.cols, pr.batch, 64, b_box_rows, 1);
    if (rc) return rc;
  } else {
    la.tm_b2 = la.tm_b;
  }
  if (!e.transposed_out) {
    rc = encode_map(&la.tm_d, out, out_cols, out_rows, pr.batch, 64, 32, 1);
    if (rc) return rc;
  } else {
    la.tm_d = la.tm_a;
  }

  KernelParams& p = la.p;
  p.m = static_cast<int>(pr.rows);
  p.n = static_cast<int>(pr.cols);
  p.k = static_cast<int>(pr.k);
  p.batch = static_cast<int>(pr.batch);
  p.m_tiles = plan.m_tiles;
  p.n_tiles = plan.n_tiles;
  p.k_blocks = plan.k_blocks;
  p.splits = plan.splits;
  p.kb_per_split = plan.kb_per_split;
  p.split_from_tile = plan.split_from_tile;
  p.narrow_from_tile = plan.narrow_from_tile;
  p.cluster_split = plan.cluster_split;
  p.stream_k = plan.stream_k;
  p.kb_per_cta = plan.kb_per_cta;
  p.idesc_narrow = make_idesc(is_bf16, 128 * e.cta_group, e.tile_n / 2);
  p.total_units = plan.total_units;
  p.group_m = plan.group_m;
  p.is_bf16 = is_bf16;
  p.idesc = make_idesc(is_bf16, 128 * e.cta_group, e.tile_n);
  // Hints are given for a/bt as the caller passed them.
  p.l2_hint_a = static_cast<uint32_t>(c.swap_ab ? c.l2_hint_b : c.l2_hint_a);
  p.l2_hint_b = static_cast<uint32_t>(c.swap_ab ? c.l2_hint_a : c.l2_hint_b);
  p.bias = bias;
  p.out = out;
  p.out_ld = out_cols;               // direct stores: out[batch][col][row], row-major [M][N]
  p.out_batch_stride = out_rows * out_cols;
  p.status = status;
  p.timeout_ns = static_cast<unsigned long long>(g_timeout_ns.load());
  p.debug_flags = g_debug_flags.load();
  p.l2_prefetch = c.l2_prefetch;
  p.early_prefetch = c.early_prefetch;
  // The early prefetch covers the operand that carries the bytes (a weight against a few rows of
  // activations); both when they are within a factor of four of each other.
  p.early_operands = (pr.rows * 4 >= pr.cols ? 1 : 0) | (pr.cols * 4 >= pr.rows ? 2 : 0);
  p.div_tiles_per_batch = FastDiv::make(static_cast<uint32_t>(plan.m_tiles) * static_cast<uint32_t>(plan.n_tiles));
  p.div_group_size = FastDiv::make(static_cast<uint32_t>(plan.group_m) * static_cast<uint32_t>(plan.n_tiles));
  p.div_group_m = FastDiv::make(static_cast<uint32_t>(plan.group_m));
  p.div_last_group_rows = FastDiv::make(static_cast<uint32_t>(plan.m_tiles % plan.group_m));
  p.div_splits = FastDiv::make(static_cast<uint32_t>(plan.splits));
  {
    int per_unit = e.cta_group * (plan.cluster_split > 0 ? plan.cluster_split : 1), log2 = 0;
    while ((1 << log2) < per_unit) ++log2;
    p.ctas_per_unit_log2 = log2;
  }
  p.stages = e.stages;
  if (plan.cluster_split > 0) {
    // Cluster split-K: every CTA receives the other k-splits' partials of the columns it owns in an
    // inbox of shared memory.  The inbox takes the top of the ring region; the ring gives up the
    // slots it covers as long as three remain, otherwise the inbox overlays live slots and the
    // kernel holds the partials back until the whole cluster is done with its MMAs.
    const int csk = plan.cluster_split;
    const int slice_cols = e.tile_n / csk;
    const int chunk_cols = e.tile_n < 32 ? e.tile_n : 32;
    const int slots = (slice_cols >= chunk_cols) ? csk - 1 : csk;
    const int inbox_bytes = slots * 128 * slice_cols * 4;
    const int stage_bytes = e.kb_per_slot * (128 * 64 * 2 + (e.tile_n / e.cta_group) * 64 * 2);  // one ring slot
    const int ring_bytes = e.stages * stage_bytes;
    if (inbox_bytes > ring_bytes) {
      return fail(AYLA_B200_E_UNSUPPORTED, "cluster_split: the %d-byte inbox does not fit the %d-byte ring", inbox_bytes,
                  ring_bytes);
    }
    const int free_stages = (ring_bytes - inbox_bytes) / stage_bytes;
    p.inbox_tx = static_cast<uint32_t>(inbox_bytes);
    p.inbox_offset = static_cast<uint32_t>(ring_bytes - inbox_bytes);
    if (free_stages >= 3 && (g_debug_flags.load() & 2) == 0) {
      p.stages = free_stages;
      p.inbox_in_ring = 0;
    } else {
      p.inbox_in_ring = 1;
    }
  }
  p.tile_rows = plan.tile_rows;
  p.act = activation;
  p.mul = mul;
  p.mul_per_row = mul_per_row;
  // One stage receives this CTA's rows of the row operand and its share of the column
  // operand; the leader of a pair counts both CTAs' bytes.
  p.stage_tx = static_cast<uint32_t>((a_box_rows + b_stage_rows) * 128 * e.cta_group);
  if (plan.slabs > 0) {
    const size_t need = workspace_bytes_for(plan);
    if (workspace == nullptr || workspace_bytes < need) {
      return fail(AYLA_B200_E_WORKSPACE, "this schedule (split_k=%d, stream_k=%d) needs a workspace of %zu bytes, got %zu",
                  plan.splits, plan.stream_k, need, workspace == nullptr ? size_t(0) : workspace_bytes);
    }
    if (!aligned16(workspace)) {
      return fail(AYLA_B200_E_INVALID, "workspace must be 16-byte aligned");
    }
    p.counters = reinterpret_cast<unsigned*>(workspace);
    p.ws = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + counter_bytes_for(plan));
  }
#ifdef AYLA_B200_TRACE
  // Tuning builds: a schedule that needs no scratch lends the workspace to the per-CTA cycle counters.
  if (plan.slabs == 0 && workspace != nullptr && workspace_bytes >= (4096 + static_cast<size_t>(plan.grid) * 64) * 8) {
    p.trace = reinterpret_cast<long long*>(workspace);
  }
#endif
  la.grid = plan.grid;
  la.cluster_x = plan.cluster_split * e.cta_group;
  la.overlap = g_launch_overlap.load();
  la.stream = stream;
  const cudaError_t err = e.launch(la);
  if (err != cudaSuccess) {
    return fail(AYLA_B200_E_CUDA, "kernel launch failed: %s", cudaGetErrorString(err));
  }
  return AYLA_B200_OK;
}

// ----------------------------------------------------- built-in split-K scratch
//
// Scratch for ayla_b200_gemm_static_scratch: a fixed array in device memory that is
// part of the loaded library image on every GPU, so that entry point never has to
// ask anyone for memory.  In host code `g_static_scratch` is only a handle for
// the runtime (not a device address); the address a kernel can use comes from
// cudaGetSymbolAddress, looked up once per device with that device current.
static __device__ __align__(256) unsigned char g_static_scratch[AYLA_B200_STATIC_SCRATCH_BYTES];

std::mutex g_scratch_mutex;
void* g_scratch_ptr[kMaxDevices] = {};

int static_scratch_for_current_device(int device, void** out) {
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_ptr[device] == nullptr) {
    void* ptr = nullptr;
    const cudaError_t err = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (err != cudaSuccess || ptr == nullptr) {
      return fail(AYLA_B200_E_CUDA, "cudaGetSymbolAddress(static scratch) on device %d: %s", device,
                  cudaGetErrorString(err));
    }
    g_scratch_ptr[device] = ptr;
  }
  *out = g_scratch_ptr[device];
  return AYLA_B200_OK;
}

}  // namespace
}  // namespace ayla_b200

using namespace ayla_b200;

extern "C" {

int ayla_b200_init(int device) {
  if (device < 0 || device >= kMaxDevices) {
    return fail(AYLA_B200_E_INVALID, "device %d out of range", device);
  }
  std::lock_guard<std::mutex> lock(g_init_mutex);
  if (g_devices[device].ready.load(std::memory_order_acquire)) return AYLA_B200_OK;
  int prev = -1;
  cudaError_t err = cudaGetDevice(&prev);
  if (err != cudaSuccess) return fail(AYLA_B200_E_CUDA, "cudaGetDevice: %s", cudaGetErrorString(err));
  err = cudaSetDevice(device);
  if (err != cudaSuccess) return fail(AYLA_B200_E_CUDA, "cudaSetDevice: %s", cudaGetErrorString(err));
  int rc = AYLA_B200_OK;
  do {
    cudaDeviceProp prop;
    err = cudaGetDeviceProperties(&prop, device);
    if (err != cudaSuccess) {
      rc = fail(AYLA_B200_E_CUDA, "cudaGetDeviceProperties: %s", cudaGetErrorString(err));
      break;
    }
    if (prop.major != 10) {
      rc = fail(AYLA_B200_E_UNSUPPORTED, "device %d is sm_%d%d; this library is sm_100a only", device,
                prop.major, prop.minor);
      break;
    }
    if (g_encode_tiled == nullptr) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult qres;
      err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
      if (err != cudaSuccess || fn == nullptr || qres != cudaDriverEntryPointSuccess) {
        rc = fail(AYLA_B200_E_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
        break;
      }
      g_encode_tiled = reinterpret_cast<PFN_cuTensorMapEncodeTiled>(fn);
    }
    const Registry& reg = registry();
    for (int i = 0; i < reg.count; ++i) {
      const KernelEntry& e = reg.entries[i];
      err = cudaFuncSetAttribute(e.func, cudaFuncAttributeMaxDynamicSharedMemorySize, e.smem_bytes);
      if (err != cudaSuccess) {
        rc = fail(AYLA_B200_E_CUDA, "cudaFuncSetAttribute(smem=%d) for variant %d: %s", e.smem_bytes, i,
                  cudaGetErrorString(err));
        break;
      }
    }
    if (rc) break;
    {
      // Resolve the built-in scratch array here as well, with `device` current: the query loads the
      // library's device image if nothing has yet, which is better done at set-up than inside the
      // first ayla_b200_gemm_static_scratch call.
      void* scratch = nullptr;
      rc = static_scratch_for_current_device(device, &scratch);
      if (rc) break;
    }
    g_devices[device].sm_count = prop.multiProcessorCount;
    g_devices[device].ready.store(true, std::memory_order_release);
  } while (false);
  if (prev >= 0 && prev != device) cudaSetDevice(prev);
  return rc;
}

int ayla_b200_default_config(int op, int dtype, int64_t batch, int64_t m, int64_t n, int64_t k,
                             ayla_b200_config* cfg_out) {
  if (cfg_out == nullptr) return fail(AYLA_B200_E_INVALID, "cfg_out is null");
  const int rc = check_shape(op, dtype, batch, m, n, k);
  if (rc) return rc;
  int sm_count = 148;
  int dev = -1;
  if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < kMaxDevices &&
      g_devices[dev].ready.load(std::memory_order_acquire)) {
    sm_count = g_devices[dev].sm_count;
  } else {
    (void)cudaGetLastError();
  }
  default_config(batch, m, n, k, sm_count, cfg_out);
  return AYLA_B200_OK;
}

int ayla_b200_config_valid(const ayla_b200_config* cfg, int op, int dtype, int64_t batch, int64_t m,
                           int64_t n, int64_t k) {
  if (cfg == nullptr) return fail(AYLA_B200_E_INVALID, "cfg is null");
  int rc = check_shape(op, dtype, batch, m, n, k);
  if (rc) return rc;
  rc = check_config(*cfg, false);
  if (rc) return rc;
  Plan plan{};
  const int epi = (op == AYLA_B200_OP_ADDMM) ? EPI_BIAS : EPI_PLAIN;
  return make_plan(*cfg, epi, batch, cfg->swap_ab ? n : m, cfg->swap_ab ? m : n, k, 148, &plan);
}

size_t ayla_b200_workspace_bytes(const ayla_b200_config* cfg, int op, int64_t batch, int64_t m,
                                 int64_t n, int64_t k) {
  if (cfg == nullptr || check_config(*cfg, false) != AYLA_B200_OK) return 0;
  if (batch <= 0 || m <= 0 || n <= 0 || k <= 0) return 0;
  Plan plan{};
  const int epi = (op == AYLA_B200_OP_ADDMM) ? EPI_BIAS : EPI_PLAIN;
  if (make_plan(*cfg, epi, batch, cfg->swap_ab ? n : m, cfg->swap_ab ? m : n, k, 148, &plan)) return 0;
  return workspace_bytes_for(plan);
}

size_t ayla_b200_workspace_counter_bytes(const ayla_b200_config* cfg, int op, int64_t batch,
                                         int64_t m, int64_t n, int64_t k) {
  if (cfg == nullptr || check_config(*cfg, false) != AYLA_B200_OK) return 0;
  if (batch <= 0 || m <= 0 || n <= 0 || k <= 0) return 0;
  Plan plan{};
  const int epi = (op == AYLA_B200_OP_ADDMM) ? EPI_BIAS : EPI_PLAIN;
  if (make_plan(*cfg, epi, batch, cfg->swap_ab ? n : m, cfg->swap_ab ? m : n, k, 148, &plan)) return 0;
  return counter_bytes_for(plan);
}

int ayla_b200_gemm(int op, int dtype, const void* bias, const void* a, const void* bt, void* out,
                   int64_t batch, int64_t m, int64_t n, int64_t k, const ayla_b200_config* cfg,
                   void* workspace, size_t workspace_bytes, uint32_t* status, void* stream) {
  return ayla_b200_gemm_act(op, dtype, AYLA_B200_ACT_NONE, bias, a, bt, out, batch, m, n, k, cfg, workspace,
                            workspace_bytes, status, stream);
}

int ayla_b200_gemm_act(int op, int dtype, int activation, const void* bias, const void* a, const void* bt,
                       void* out, int64_t batch, int64_t m, int64_t n, int64_t k,
                       const ayla_b200_config* cfg, void* workspace, size_t workspace_bytes,
                       uint32_t* status, void* stream) {
  return ayla_b200_gemm_act_mul(op, dtype, activation, bias, a, bt, nullptr, out, batch, m, n, k, cfg, workspace,
                                workspace_bytes, status, stream);
}

static int gemm_fused(int op, int dtype, int activation, const void* bias, const void* a, const void* bt,
                      const void* mul, int mul_per_row, void* out, int64_t batch, int64_t m, int64_t n, int64_t k,
                      const ayla_b200_config* cfg, void* workspace, size_t workspace_bytes, uint32_t* status,
                      void* stream);

int ayla_b200_gemm_act_mul(int op, int dtype, int activation, const void* bias, const void* a, const void* bt,
                           const void* mul, void* out, int64_t batch, int64_t m, int64_t n, int64_t k,
                           const ayla_b200_config* cfg, void* workspace, size_t workspace_bytes,
                           uint32_t* status, void* stream) {
  if (mul != nullptr && !aligned16(mul)) {
    return fail(AYLA_B200_E_UNSUPPORTED, "mul must be 16-byte aligned");
  }
  return gemm_fused(op, dtype, activation, bias, a, bt, mul, 0, out, batch, m, n, k, cfg, workspace,
                    workspace_bytes, status, stream);
}

int ayla_b200_gemm_act_rowmul(int op, int dtype, int activation, const void* bias, const void* a, const void* bt,
                              const void* row_mul, void* out, int64_t batch, int64_t m, int64_t n, int64_t k,
                              const ayla_b200_config* cfg, void* workspace, size_t workspace_bytes,
                              uint32_t* status, void* stream) {
  if (row_mul == nullptr || (reinterpret_cast<uintptr_t>(row_mul) & 1) != 0) {
    return fail(AYLA_B200_E_INVALID, "row_mul must be a non-null, 2-byte aligned pointer");
  }
  return gemm_fused(op, dtype, activation, bias, a, bt, row_mul, 1, out, batch, m, n, k, cfg, workspace,
                    workspace_bytes, status, stream);
}

static int gemm_fused(int op, int dtype, int activation, const void* bias, const void* a, const void* bt,
                      const void* mul, int mul_per_row, void* out, int64_t batch, int64_t m, int64_t n, int64_t k,
                      const ayla_b200_config* cfg, void* workspace, size_t workspace_bytes, uint32_t* status,
                      void* stream) {
  int rc = check_shape(op, dtype, batch, m, n, k);
  if (rc) return rc;
  if (activation < AYLA_B200_ACT_NONE || activation > AYLA_B200_ACT_GELU_TANH) {
    return fail(AYLA_B200_E_INVALID, "unknown activation %d", activation);
  }
  if (a == nullptr || bt == nullptr || out == nullptr) {
    return fail(AYLA_B200_E_INVALID, "a, bt and out must be non-null");
  }
  if (op == AYLA_B200_OP_ADDMM && bias == nullptr) {
    return fail(AYLA_B200_E_INVALID, "addmm needs a bias pointer");
  }
  if (!aligned16(a) || !aligned16(bt) || !aligned16(out)) {
    return fail(AYLA_B200_E_UNSUPPORTED, "a, bt and out must be 16-byte aligned");
  }
  DeviceState* ds = nullptr;
  int dev = -1;
  rc = current_device_state(&ds, &dev);
  if (rc) return rc;

  ayla_b200_config c;
  if (cfg != nullptr) {
    c = *cfg;
  } else {
    default_config(batch, m, n, k, ds->sm_count, &c);
  }
  rc = check_config(c, false);
  if (rc) return rc;

  Problem pr;
  pr.k = k;
  pr.batch = batch;
  if (c.swap_ab) {
    pr.rows = n;
    pr.cols = m;
    pr.row_operand = bt;
    pr.col_operand = a;
  } else {
    pr.rows = m;
    pr.cols = n;
    pr.row_operand = a;
    pr.col_operand = bt;
  }
  const int epi = (op == AYLA_B200_OP_ADDMM) ? EPI_BIAS : EPI_PLAIN;
  Plan plan{};
  rc = make_plan(c, epi, batch, pr.rows, pr.cols, k, ds->sm_count, &plan, (activation != 0 || mul != nullptr) ? 1 : 0);
  if (rc) return rc;
  return launch_plan(plan, c, pr, dtype == AYLA_B200_BF16 ? 1 : 0, bias, nullptr, out, m, n, workspace,
                     workspace_bytes, status, reinterpret_cast<cudaStream_t>(stream), activation, mul, mul_per_row);
}

int ayla_b200_gemm_static_scratch(int op, int dtype, const void* bias, const void* a, const void* bt,
                                  void* out, int64_t batch, int64_t m, int64_t n, int64_t k,
                                  const ayla_b200_config* cfg, uint32_t* status, void* stream) {
  int rc = check_shape(op, dtype, batch, m, n, k);
  if (rc) return rc;
  if (a == nullptr || bt == nullptr || out == nullptr) {
    return fail(AYLA_B200_E_INVALID, "a, bt and out must be non-null");
  }
  if (op == AYLA_B200_OP_ADDMM && bias == nullptr) {
    return fail(AYLA_B200_E_INVALID, "addmm needs a bias pointer");
  }
  if (!aligned16(a) || !aligned16(bt) || !aligned16(out)) {
    return fail(AYLA_B200_E_UNSUPPORTED, "a, bt and out must be 16-byte aligned");
  }
  DeviceState* ds = nullptr;
  int dev = -1;
  rc = current_device_state(&ds, &dev);
  if (rc) return rc;
  ayla_b200_config c;
  if (cfg != nullptr) {
    c = *cfg;
  } else {
    default_config(batch, m, n, k, ds->sm_count, &c);
  }
  rc = check_config(c, false);
  if (rc) return rc;
  Problem pr;
  pr.k = k;
  pr.batch = batch;
  pr.rows = c.swap_ab ? n : m;
  pr.cols = c.swap_ab ? m : n;
  pr.row_operand = c.swap_ab ? bt : a;
  pr.col_operand = c.swap_ab ? a : bt;
  const int epi = (op == AYLA_B200_OP_ADDMM) ? EPI_BIAS : EPI_PLAIN;
  Plan plan{};
  rc = make_plan(c, epi, batch, pr.rows, pr.cols, k, ds->sm_count, &plan);
  if (rc) return rc;
  const size_t need = workspace_bytes_for(plan);
  if (need > static_cast<size_t>(AYLA_B200_STATIC_SCRATCH_BYTES)) {
    return fail(AYLA_B200_E_WORKSPACE,
                "this schedule needs %zu bytes of split-K scratch; the built-in array holds %zu "
                "(use ayla_b200_gemm with a caller workspace, or a smaller split_k)",
                need, static_cast<size_t>(AYLA_B200_STATIC_SCRATCH_BYTES));
  }
  void* scratch = nullptr;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (need > 0) {
    rc = static_scratch_for_current_device(dev, &scratch);
    if (rc) return rc;
    // The array keeps whatever the previous call left behind.  Only the arrival
    // counters must start at zero; partial sums are fully rewritten before they are read.
    const cudaError_t err = cudaMemsetAsync(scratch, 0, static_cast<size_t>(plan.row_tiles) * 4, s);
    if (err != cudaSuccess) {
      return fail(AYLA_B200_E_CUDA, "clearing the split-K counters: %s", cudaGetErrorString(err));
    }
  }
  return launch_plan(plan, c, pr, dtype == AYLA_B200_BF16 ? 1 : 0, bias, nullptr, out, m, n, scratch, need,
                     status, s);
}

int ayla_b200_swiglu(int dtype, const void* x, const void* w_gate, const void* w_up, void* out,
                     int64_t m, int64_t n, int64_t k, const ayla_b200_config* cfg, uint32_t* status,
                     void* stream) {
  int rc = check_shape(AYLA_B200_OP_MM, dtype, 1, m, n, k);
  if (rc) return rc;
  if (x == nullptr || w_gate == nullptr || w_up == nullptr || out == nullptr) {
    return fail(AYLA_B200_E_INVALID, "x, w_gate, w_up and out must be non-null");
  }
  if (!aligned16(x) || !aligned16(w_gate) || !aligned16(w_up) || !aligned16(out)) {
    return fail(AYLA_B200_E_UNSUPPORTED, "x, w_gate, w_up and out must be 16-byte aligned");
  }
  DeviceState* ds = nullptr;
  int dev = -1;
  rc = current_device_state(&ds, &dev);
  if (rc) return rc;
  ayla_b200_config c;
  if (cfg != nullptr) {
    c = *cfg;
  } else {
    memset(&c, 0, sizeof(c));
    c.cta_group = (m >= 256) ? 2 : 1;
    c.group_m = 8;
    c.l2_hint_a = 2;  // x is re-read by every column tile,
    c.l2_hint_b = 1;  // the weights stream through once
  }
  c.tile_n = 256;
  c.split_k = 1;
  c.swap_ab = 0;
  rc = check_config(c, true);
  if (rc) return rc;
  Problem pr;
  pr.rows = m;
  pr.cols = n;
  pr.k = k;
  pr.batch = 1;
  pr.row_operand = x;
  pr.col_operand = w_gate;
  Plan plan{};
  rc = make_plan(c, EPI_SWIGLU, 1, m, n, k, ds->sm_count, &plan);
  if (rc) return rc;
  return launch_plan(plan, c, pr, dtype == AYLA_B200_BF16 ? 1 : 0, nullptr, w_up, out, m, n, nullptr, 0,
                     status, reinterpret_cast<cudaStream_t>(stream));
}

// The listing covers the variants without the activation epilogue; each of them except the
// SwiGLU pair exists a second time with it.
int ayla_b200_kernel_count(void) { return registry().base_count; }

int ayla_b200_kernel_info(int i, int32_t* tile_n, int32_t* cta_group, int32_t* epilogue,
                          int32_t* transposed_out, int32_t* stages, int32_t* smem_bytes) {
  const Registry& reg = registry();
  if (i < 0 || i >= reg.base_count) return fail(AYLA_B200_E_INVALID, "variant index %d out of range", i);
  const KernelEntry& e = reg.entries[i];
  if (tile_n) *tile_n = e.tile_n;
  if (cta_group) *cta_group = e.cta_group;
  if (epilogue) *epilogue = e.epilogue;
  if (transposed_out) *transposed_out = e.transposed_out;
  if (stages) *stages = e.stages;
  if (smem_bytes) *smem_bytes = e.smem_bytes;
  return AYLA_B200_OK;
}

void ayla_b200_set_wait_timeout_ms(int64_t ms) {
  if (ms < 1) ms = 1;
  g_timeout_ns.store(ms * 1000000ll);
}

int ayla_b200_copy_2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes,
                      size_t rows, void* stream) {
  if (dst == nullptr || src == nullptr) return fail(AYLA_B200_E_INVALID, "dst and src must be non-null");
  if (width_bytes == 0 || rows == 0) return AYLA_B200_OK;
  if (dst_pitch < width_bytes || src_pitch < width_bytes) {
    return fail(AYLA_B200_E_INVALID, "pitches must be at least the row width");
  }
  const cudaError_t err = cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, rows,
                                            cudaMemcpyDeviceToDevice, reinterpret_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) return fail(AYLA_B200_E_CUDA, "cudaMemcpy2DAsync: %s", cudaGetErrorString(err));
  return AYLA_B200_OK;
}

void ayla_b200_debug_set_flags(int flags) { g_debug_flags.store(flags); }

void ayla_b200_set_launch_overlap(int enabled) { g_launch_overlap.store(enabled ? 1 : 0); }

const char* ayla_b200_last_error(void) { return g_last_error.c_str(); }

const char* ayla_b200_version(void) { return "ayla_b200 0.1 (sm_100a, tcgen05)"; }

}  // extern "C"
