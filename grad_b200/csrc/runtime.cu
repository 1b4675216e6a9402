// Host side of libgradb200.so: argument validation, tile / split-K selection, tensor-map encoding and
// dispatch for the entry points declared in include/gradb200.h.  This is the counterpart of the
// wrappers in grad's src/gpu/gpu.zig (`matmul` :642-679, `matmulPacked` :1036-1064, `forwardPlan`
// :890-913, `convImplicitWeightGrad` :983-1022, `convF32Forward` :789-826): it decides how a product is
// cut into tiles and K parts; the kernels it launches live in gemm_sm100.cu and gemm_f32.cu.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>
#include <mutex>

#include "../../include/gradb200.h"
#include "gemm_sm100.cuh"

namespace gb {
cudaError_t launch_gemm_f32(const GemmParams& p, cudaStream_t stream);
bool conv_direct_applies(const GemmParams& p);
cudaError_t launch_conv_direct(const GemmParams& p, int sm_count, cudaStream_t stream);
bool conv_direct_wgrad_applies(const GemmParams& p);
uint32_t conv_direct_wgrad_blocks(const GemmParams& p, int sm_count);
cudaError_t launch_conv_direct_wgrad(const GemmParams& p, uint32_t blocks, cudaStream_t stream);
cudaError_t launch_affine_expand(const float* mean, const float* inv_std, const float* gamma, const float* beta, uint16_t* scale, uint16_t* shift,
                                 uint32_t c, cudaStream_t stream);
}

struct gb_handle;

namespace {

using gb::GemmParams;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
      return (EncodeTiledFn) nullptr;
    return (EncodeTiledFn)ptr;
  }();
  return fn;
}

// Tuning knobs, read from the environment once per process.  Each one switches a plan back to the plan it
// replaced, which is how the two were compared on the device; none is needed in normal use.
struct Knobs {
  int group_m = 0;               // GB_GROUP_M=n: height of the tile rasterisation band (default 8)
  bool no_pair = false;          // GB_NO_PAIR: single-CTA tiles only
  bool no_tma_store = false;     // GB_NO_TMA_STORE: results leave by per-lane stores
  bool no_column_stages = false; // GB_NO_COLUMN_STAGES: one stage per tap instead of one per tap column
  bool no_direct_conv = false;   // GB_NO_DIRECT_CONV: the stem goes through the gathered tensor plan
  bool no_strided_tma = false;   // GB_NO_STRIDED_TMA: strided forward / weight-gradient patches are gathered
  bool no_dgrad_classes = false; // GB_NO_DGRAD_CLASSES: a strided input gradient is one gathered product
  bool no_wide_stages = false;   // GB_NO_WIDE_STAGES: weight gradients keep one K block per stage
  bool no_fused_classes = false; // GB_NO_FUSED_CLASSES: one launch per parity class of a strided input gradient
  bool no_stem_lines = false;    // GB_NO_STEM_LINES: the 3-channel stem keeps the FMA kernel for its forward pass
  bool no_plan_cache = false;    // GB_NO_PLAN_CACHE: every call plans from scratch
  int force_bn = 0;              // GB_FORCE_BN=n: tile width of a dense single-CTA product (with GB_FORCE_SPLITS: its K split)
  int force_splits = 0;
  // Host-requested failure injection for the time-out path (tests only): the first GB_TEST_DROP_CALLS (default 1)
  // single-CTA tensor launches of each handle leave out the copies of K block GB_TEST_DROP_KBLOCK, and bounded waits
  // give up after GB_TEST_SPIN_LIMIT polls instead of about a second's worth.
  uint32_t test_spin_limit = 0, test_drop_kblock = 0, test_drop_calls = 0;
};
const Knobs& knobs() {
  static const Knobs k = [] {
    Knobs v;
    if (const char* g = getenv("GB_GROUP_M")) v.group_m = std::max(1, atoi(g));
    v.no_pair = getenv("GB_NO_PAIR") != nullptr;
    v.no_tma_store = getenv("GB_NO_TMA_STORE") != nullptr;
    v.no_column_stages = getenv("GB_NO_COLUMN_STAGES") != nullptr;
    v.no_direct_conv = getenv("GB_NO_DIRECT_CONV") != nullptr;
    v.no_strided_tma = getenv("GB_NO_STRIDED_TMA") != nullptr;
    v.no_dgrad_classes = getenv("GB_NO_DGRAD_CLASSES") != nullptr;
    v.no_wide_stages = getenv("GB_NO_WIDE_STAGES") != nullptr;
    v.no_fused_classes = getenv("GB_NO_FUSED_CLASSES") != nullptr;
    v.no_stem_lines = getenv("GB_NO_STEM_LINES") != nullptr;
    v.no_plan_cache = getenv("GB_NO_PLAN_CACHE") != nullptr;
    if (const char* g = getenv("GB_FORCE_BN")) v.force_bn = atoi(g);
    if (const char* g = getenv("GB_FORCE_SPLITS")) v.force_splits = atoi(g);
    if (const char* g = getenv("GB_TEST_SPIN_LIMIT")) v.test_spin_limit = (uint32_t)std::max(1, atoi(g));
    if (const char* g = getenv("GB_TEST_DROP_KBLOCK")) {
      v.test_drop_kblock = (uint32_t)std::max(0, atoi(g)) + 1;
      v.test_drop_calls = 1;
      if (const char* c = getenv("GB_TEST_DROP_CALLS")) v.test_drop_calls = (uint32_t)std::max(0, atoi(c));
    }
    return v;
  }();
  return k;
}

uint32_t ceil_div(uint32_t a, uint32_t b) { return (a + b - 1) / b; }
uint32_t elem_size(uint32_t dtype) { return dtype == GB_BF16 ? 2u : 4u; }
bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

// Encodes a tiled map with 128-byte swizzle.  dims/strides/box follow the driver's convention: dims[0] is
// the contiguous one, strides (bytes) start at dims[1].
// `oob_nan`: elements outside the tensor arrive as NaN instead of zero (for an operand that is transformed after it lands and
// whose padding must come out as exactly zero: see GemmParams::xform).
bool encode_map(CUtensorMap* map, bool bf16, const void* base, uint32_t rank, const uint64_t* dims, const uint64_t* strides_bytes,
                const uint32_t* box, bool swizzle_32b_chunks = false, const uint32_t* elem_strides = nullptr, bool swizzle_64b = false,
                bool oob_nan = false) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  cuuint64_t gdims[5];
  cuuint64_t gstrides[4];
  cuuint32_t gbox[5], estr[5];
  for (uint32_t i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = elem_strides ? elem_strides[i] : 1;
    if (i + 1 < rank) gstrides[i] = strides_bytes[i];
  }
  const CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, rank, const_cast<void*>(base),
                        gdims, gstrides, gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle_64b ? CU_TENSOR_MAP_SWIZZLE_64B
                                    : (swizzle_32b_chunks ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B),
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        oob_nan ? CU_TENSOR_MAP_FLOAT_OOB_FILL_NAN_REQUEST_ZERO_FMA : CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Ordered batch-norm statistics: 8 epilogue warps x 4 chunks x 32 lanes x (sum, squares) floats per CTA.
constexpr size_t kStatsPartialBytesPerCta = 8 * 4 * 64 * sizeof(float);

enum LaunchKind : uint32_t { kLaunchNone, kLaunchDirect, kLaunchDirectWgrad, kLaunchEmptyK, kLaunchTensor, kLaunchF32 };

struct Plan {
  GemmParams p;
  CUtensorMap tmap_a, tmap_b, tmap_c;
  LaunchKind launch = kLaunchNone;   // set by prepare_plan: which kernel runs ...
  bool reduce = false;               // ... and whether the split-K reduce follows it
  gb_plan_info info = {};            // what gb_last_plan reports after the launch
  bool direct = false;      // forward convolution with very few input channels: the FMA kernel of conv_direct.cu
  bool stats_ordered = false;         // statistics through per-CTA partials in the workspace and an ordered combine
  uint32_t stats_ctas = 0;
  uint32_t direct_wgrad_blocks = 0;   // > 0: weight gradient of such a layer by the FMA kernel, this many position ranges
  size_t direct_wgrad_bytes = 0;      // ... when the workspace holds their partial matrices
  bool tensor = false;      // tcgen05 path, else strict-f32
  size_t workspace = 0;     // bytes of split-K partials
};

struct PlanKey {
  uint32_t kind, pad;
  unsigned char desc[72];
  uint64_t ptr[11];
  uint64_t hash;     // over the bytes before it
};
struct CachedPlan {
  PlanKey key;
  Plan plan;
  uint64_t stamp;
};

}  // namespace

struct gb_handle {
  int device = 0;
  int sm_count = 0;
  int last_cuda = 0;
  uint32_t* status = nullptr;   // device word the kernels report bounded-wait failures into
  uint32_t test_drops_left = 0; // fault injection requested through the environment: calls that still drop a K block
  gb_plan_info last_plan = {};
  std::vector<CachedPlan> cache;   // prepared plans of recent calls
  uint64_t cache_clock = 0, cache_hits = 0;
};

namespace {

int cuda_fail(gb_handle* h, cudaError_t e) {
  if (h) h->last_cuda = (int)e;
  return GB_ERR_CUDA;
}

// Dense operand stored as `lines` rows of `inner` contiguous elements with pitch ld.
struct DenseOperand {
  const void* base;
  uint32_t dtype, lines, inner, ld;
  uint64_t batch_stride;
  bool mn_major;            // the contiguous (inner) index is the MN index
  uint32_t outer = 1;       // second batch level: count and stride in elements
  uint64_t outer_stride = 0;
};

void fill_dense_gather(gb::GatherDesc& g, const DenseOperand& o) {
  g.base = o.base;
  g.batch_stride = o.batch_stride;
  g.source = gb::kSrcDense;
  g.src_is_bf16 = o.dtype == GB_BF16;
  g.ld = o.ld;
  g.lines_total = o.lines;
  g.inner_total = o.inner;
  g.mn_major = o.mn_major;
}

// Tries to describe a dense operand by a TMA map {inner, lines, batch, 1}; false means "gather it".
bool dense_tma(CUtensorMap* map, const DenseOperand& o, bool smem_bf16, uint32_t batch, uint32_t tile_mn, uint32_t epl, uint32_t k_mul = 1) {
  const uint32_t es = smem_bf16 ? 2 : 4;
  if ((o.dtype == GB_BF16) != smem_bf16) return false;
  if (!aligned16(o.base) || ((uint64_t)o.ld * es) % 16 != 0) return false;
  if (batch > 1 && (o.batch_stride == 0 || (o.batch_stride * es) % 16 != 0)) return false;
  if (o.outer > 1 && (o.outer_stride == 0 || (o.outer_stride * es) % 16 != 0)) return false;
  // Every operand map has four dimensions (the kernel issues one form of copy); a dense one ends in the outer batch
  // level, an extent of 1 when there is none.
  const uint64_t dims[4] = {o.inner, o.lines, batch, o.outer};
  const uint64_t batch_bytes = batch > 1 ? o.batch_stride * es : (uint64_t)o.ld * es * std::max<uint64_t>(o.lines, 1);
  const uint64_t strides[3] = {(uint64_t)o.ld * es, batch_bytes, o.outer > 1 ? o.outer_stride * es : batch_bytes * batch};
  // K-major: box = 128 bytes of K x tile_mn lines.  MN-major: box = 128 bytes of MN x epl K lines.
  const uint32_t box[4] = {epl, o.mn_major ? epl * k_mul : tile_mn, 1, 1};
  if (box[1] > 256) return false;
  // MN-major 32-bit tiles must use the 32-byte-chunk flavour of the 128-byte swizzle.
  return encode_map(map, smem_bf16, o.base, 4, dims, strides, box, !smem_bf16 && o.mn_major);
}

uint32_t pick_stages(uint32_t bn) {
  const uint32_t stage = 128 * 128 + bn * 128;
  return std::min<uint32_t>(8, (227 * 1024 - 2048) / stage);
}

// Estimated cycles of a product cut into 128- (single CTA) or 256-row (CTA pair) tiles of width bn.  Per K
// block an SM needs max(MMA time, shared-memory fill time): 128 x bn x 64 MACs at 4096 MACs/clk, and
// 16 KB of A plus its lines of B at the ~48 B/clk TMA sustains per SM.  A tile also pays a fixed cost
// (barrier round trips, epilogue tail; the 512-wide tile's whole epilogue, which nothing overlaps), and
// tiles are dealt to `units` persistent CTAs (or CTA pairs) in waves.
double tile_cost(uint32_t m, uint32_t n, uint32_t batch, uint32_t k_blocks, uint32_t bn, bool pair, uint32_t sms) {
  const uint32_t rows = pair ? 256 : 128, units = pair ? sms / 2 : sms;
  const uint64_t tiles = (uint64_t)ceil_div(m, rows) * ceil_div(n, bn) * batch;
  if (tiles == 0 || units == 0) return 0.0;
  const double b_lines = pair ? bn / 2.0 : bn;
  // One tcgen05.mma costs its issuing thread 45-65 cycles whatever its N, so narrow tiles are issue-bound.
  const double fill = (16384.0 + b_lines * 128.0) / 48.0, mma = 4.0 * std::max(bn / 2.0, 60.0);
  const double per_tile = k_blocks * std::max(fill, mma) + (bn > 256 ? 11000.0 : 1200.0);
  const double waves = (double)((tiles + units - 1) / units);
  // A cluster launch, its two cluster-wide syncs and the cross-CTA barrier arrivals cost a pair kernel ~1.5 us more than a
  // single-CTA one whatever the product (7.4 against 4.9 us for one K block per SM; 8.0 against 6.7 us for 8192 x 256 x 256):
  // the pair has to earn that back with its lighter shared-memory fill per K block.
  return waves * per_tile + 3000.0 + (pair ? 3000.0 : 0.0);
}

// K split a tile width would get: when its tiles leave SMs idle, about one work item per SM, each at least sixteen K
// blocks long (the role of `splits` in src/gpu/gpu.zig:664, 1000, 1041).  A split costs a second launch and a pass over
// the partials.
uint32_t split_for_width(uint32_t m, uint32_t n, uint32_t batch, uint32_t k_blocks, uint32_t bn, uint32_t sms, bool allow_split) {
  const uint32_t tiles = ceil_div(m, 128) * batch * ceil_div(n, bn);
  if (!allow_split || tiles == 0 || tiles * 2 > sms || k_blocks < 32) return 1;
  return std::max(1u, std::min(sms / tiles, k_blocks / 16));
}

// Tile width and K split for an m x n x k_blocks product on `sms` multiprocessors: the (width, split) pair with the
// lowest estimated time.  The estimate of a split product is that of its longest part plus the reduce launch and its
// pass over the partial tiles; judged by the unsplit time alone, a product with few tiles and a long K (a weight
// gradient: 2304 x 256 x 8192) took the narrowest tile -- most tiles, shortest wave -- and then ran issue-bound 64-wide
// MMAs in every part.
void pick_tiling(uint32_t m, uint32_t n, uint32_t batch, uint32_t k_blocks, uint32_t min_bn, uint32_t sms, bool allow_split,
                 uint32_t& bn, uint32_t& splits, uint32_t& kbps) {
  const uint32_t n_cap = std::max(min_bn, ceil_div(n, min_bn) * min_bn);   // n rounded up to the narrowest tile
  bn = 0;
  double best = 0.0;
  for (uint32_t cand : {256u, 128u, 64u, 32u}) {
    if (cand < min_bn || cand > n_cap) continue;
    const uint32_t parts = split_for_width(m, n, batch, k_blocks, cand, sms, allow_split);
    double cost = tile_cost(m, n, batch * parts, ceil_div(k_blocks, parts), cand, false, sms);
    if (parts > 1) cost += 4000.0 + (double)m * n * batch * parts * 4.0 / 2000.0;   // reduce launch + its read of the partials
    if (bn == 0 || cost < best) { bn = cand; best = cost; }
  }
  if (bn == 0) bn = min_bn;
  if (knobs().force_bn >= (int)min_bn && knobs().force_bn <= 256 && knobs().force_bn % 32 == 0) bn = (uint32_t)knobs().force_bn;
  splits = split_for_width(m, n, batch, k_blocks, bn, sms, allow_split);
  if (allow_split && knobs().force_splits > 0) splits = std::min<uint32_t>((uint32_t)knobs().force_splits, std::max(1u, k_blocks));
  kbps = std::max(1u, ceil_div(k_blocks, splits));
  splits = std::max(1u, ceil_div(k_blocks, kbps));
}

int finish_plan(const gb_handle* h, Plan& plan, bool allow_split, uint32_t min_bn, const gb_epilogue* ep) {
  GemmParams& p = plan.p;
  p.bias = ep ? ep->bias : nullptr;
  p.residual = ep ? ep->residual : nullptr;
  p.relu = ep && ep->activation == GB_ACT_RELU;
  p.round_tf32 = ep && (ep->flags & GB_EPILOGUE_ROUND_TF32) && !p.c_is_bf16;
  p.status = h->status;
  const gb_bn_stats* st = ep ? ep->bn_stats : nullptr;
  if (st) {
    // statistics are summed per warp over ONE column tile and over the final values: tensor path, whole 32-column chunks,
    // at most 256 columns, no K split
    if (!st->shift || !st->sums || !plan.tensor || p.n > 256 || p.n % 32 != 0 || p.batch != 1) return GB_ERR_UNSUPPORTED;
    p.stats = 1;
    p.stat_shift = st->shift;
    p.stat_sums = st->sums;
    plan.stats_ordered = st->ordered != 0;
    allow_split = false;
    min_bn = std::max<uint32_t>(min_bn, p.n <= 32 ? 32 : (p.n <= 64 ? 64 : (p.n <= 128 ? 128 : 256)));
  }
  p.epi_groups = 2;
  p.group_m = 8;
  if (knobs().group_m) p.group_m = (uint32_t)knobs().group_m;
  if (plan.tensor) {
    const uint32_t epl = p.tf32 ? 32 : 64;
    p.k_blocks_total = ceil_div(p.k, epl);
    uint32_t bn, splits, kbps;
    pick_tiling(p.m, p.n, p.batch, p.k_blocks_total, min_bn, (uint32_t)h->sm_count, allow_split, bn, splits, kbps);
    p.bn = bn;
    p.splits = splits;
    p.k_blocks_per_split = kbps;
    p.tiles_m = ceil_div(p.m, 128);
    p.tiles_n = ceil_div(p.n, bn);
    p.stages = pick_stages(bn);
  } else {
    p.k_blocks_total = ceil_div(p.k, 16);
    const uint32_t tiles = ceil_div(p.m, 64) * ceil_div(p.n, 64) * p.batch;
    uint32_t splits = 1;
    // A 16-deep K step of the CUDA-core kernel is one global-load round trip (~1 us) whatever the tile count, so a
    // product of a few tiles is as slow as its K is deep (64 x 128 x 784: 17 us in three parts): parts of two steps each,
    // as many as fill the machine, and the reduce launch (~3 us) costs less than the steps it removes.
    if (allow_split && tiles > 0 && tiles < 2u * h->sm_count && p.k_blocks_total >= 4)
      splits = std::max(1u, std::min(ceil_div(2u * h->sm_count, tiles), p.k_blocks_total / 2));
    p.k_blocks_per_split = std::max(1u, ceil_div(p.k_blocks_total, splits));
    p.splits = std::max(1u, ceil_div(p.k_blocks_total, p.k_blocks_per_split));
    p.tiles_m = ceil_div(p.m, 64);
    p.tiles_n = ceil_div(p.n, 64);
    p.bn = 64;
    p.stages = 1;
  }
  plan.workspace = p.splits > 1 ? (size_t)p.splits * p.batch * p.m * p.n * sizeof(float) : 0;
  return GB_OK;
}

// Switches a planned tensor-path product to the CTA-pair kernel (256 x bn tiles over two SMs) when both
// operands arrive by TMA, K is not split, and a pair tile has a lower estimated time than the single-CTA
// plan.  `encode_b(rows)` re-encodes B's map for the `rows` lines one CTA of the pair loads; false keeps
// the single-CTA plan.
// `mode`: 0 = by estimated time, 1 = the pair kernel whenever it can run this product, 2 = never.
// `split_k`: the pair plan may split K like the single-CTA plan does (a weight gradient: few tiles, K = all positions; a
// 256 x 256 pair tile moves 32 KB per K block and SM where the single-CTA 128 x 256 tile moves 48 KB for half the rows).
template <class EncodeB>
bool try_pair(const gb_handle* h, Plan& plan, uint32_t min_bn, EncodeB encode_b, int mode = 0, bool split_k = false) {
  GemmParams& p = plan.p;
  if (!plan.tensor || p.a_kind == gb::kGather || p.b_kind == gb::kGather || p.m <= 128 || (p.splits > 1 && !split_k)) return false;
  if (knobs().no_pair || mode == 2) return false;
  const uint32_t sms = (uint32_t)h->sm_count;
  const uint32_t n_cap = std::max(min_bn, ceil_div(p.n, min_bn) * min_bn);
  auto reduce_cost = [&](uint32_t parts) { return parts > 1 ? 4000.0 + (double)p.m * p.n * p.batch * parts * 4.0 / 2000.0 : 0.0; };
  double best = mode == 1 ? 1e300
                          : tile_cost(p.m, p.n, p.batch * p.splits, ceil_div(p.k_blocks_total, p.splits), p.bn, false, sms) + reduce_cost(p.splits);
  uint32_t pick = 0, pick_parts = 1;
  for (uint32_t cand : {512u, 256u, 128u, 64u}) {
    // a pair tile may overhang n as long as the second CTA's half still holds columns (192 columns: one 256-wide tile)
    if (cand / 2 < min_bn || (cand > n_cap && cand / 2 >= p.n)) continue;
    if (p.stats && (cand > 256 || cand < p.n)) continue;   // statistics: one column tile of at most 256 columns
    uint32_t parts = 1;
    if (split_k && !p.stats) {
      const uint32_t tiles = ceil_div(p.m, 256) * p.batch * ceil_div(p.n, cand);
      if (tiles * 2 <= sms / 2 && p.k_blocks_total >= 32) parts = std::max(1u, std::min(sms / 2 / tiles, p.k_blocks_total / 16));
      if (knobs().force_splits > 0) parts = std::min<uint32_t>((uint32_t)knobs().force_splits, std::max(1u, p.k_blocks_total));
      // K parts on a pair only for the 256-wide tile: narrower ones measured slower than the single-CTA plan with its
      // two K blocks per stage (256 x 128 pair tiles, 128 -> 128 at 16 x 16: 24.1 against 20.6 us), and the partial
      // tiles of the two-half 512-wide tile are not laid out for the reduce
      if (parts > 1 && cand != 256) continue;
    }
    const double cost = tile_cost(p.m, p.n, p.batch * parts, ceil_div(p.k_blocks_total, parts), cand, true, sms) + reduce_cost(parts);
    // a tie goes to the pair (half as many MMA instructions per row) unless it needs a K split the single-CTA plan does without
    if (cost < best || (cost == best && parts <= p.splits)) { best = cost; pick = cand; pick_parts = parts; }
  }
  if (pick == 0 || !encode_b(pick / 2)) return false;
  p.cta_pair = 1;
  p.bn = pick;
  p.tiles_m = ceil_div(p.m, 256);
  p.tiles_n = ceil_div(p.n, pick);
  p.k_blocks_per_split = std::max(1u, ceil_div(p.k_blocks_total, pick_parts));
  p.splits = std::max(1u, ceil_div(p.k_blocks_total, p.k_blocks_per_split));
  p.stages = std::min<uint32_t>(8, (227 * 1024 - 2048) / (128 * 128 + pick / 2 * 128));
  plan.workspace = p.splits > 1 ? (size_t)p.splits * p.batch * p.m * p.n * sizeof(float) : 0;
  return true;
}

void set_output(GemmParams& p, void* c, uint32_t dtype_c, uint32_t ldc, uint64_t stride_c, bool transpose_out, bool accumulate,
                const gb_epilogue* ep) {
  p.c = c;
  p.c_is_bf16 = dtype_c == GB_BF16;
  p.ldc = ldc;
  p.stride_c = stride_c;
  p.transpose_out = transpose_out;
  p.accumulate = accumulate;
  const uint32_t es = elem_size(dtype_c);
  bool vec = aligned16(c) && ((uint64_t)ldc * es) % 16 == 0 && (stride_c * es) % 16 == 0 && !transpose_out;
  if (ep && ep->bias && !aligned16(ep->bias)) vec = false;
  if (ep && ep->residual && !aligned16(ep->residual)) vec = false;
  p.vec_store = vec;
}

int validate_gemm(const gb_gemm_desc* d) {
  if (!d) return GB_ERR_INVALID;
  if (d->trans_a && d->trans_b) return GB_ERR_INVALID;   // src/gpu/gpu.zig:643
  if (d->dtype_a > GB_BF16 || d->dtype_b > GB_BF16 || d->dtype_c > GB_BF16 || d->math > GB_MATH_BF16) return GB_ERR_INVALID;
  return GB_OK;
}

int plan_gemm(const gb_handle* h, const gb_gemm_desc* d, const void* a, const void* b, void* c, const gb_epilogue* ep, Plan& plan) {
  std::memset(&plan.p, 0, sizeof(plan.p));
  GemmParams& p = plan.p;
  const uint32_t batch = std::max<uint32_t>(d->batch, 1);
  const uint32_t outer = std::max<uint32_t>(d->batch_outer, 1);
  p.m = d->m; p.n = d->n; p.k = d->k; p.batch = batch * outer;
  if (outer > 1) {
    if (d->transpose_out || d->k == 0) return GB_ERR_UNSUPPORTED;
    p.batch_inner = batch;
    p.div_batch_inner = gb::make_fastdiv_host(batch);
    p.stride_c_outer = d->stride_c_outer;
  }
  // The bf16 path is taken whenever an operand or the result is bf16, like `Gpu.matmul` (gpu.zig:644-647).
  uint32_t math = d->math;
  if (math == GB_MATH_F32 && (d->dtype_a == GB_BF16 || d->dtype_b == GB_BF16)) math = GB_MATH_BF16;
  plan.tensor = math != GB_MATH_F32;
  p.tf32 = math == GB_MATH_TF32;
  const bool smem_bf16 = math == GB_MATH_BF16;
  const uint32_t epl = p.tf32 ? 32 : 64;

  DenseOperand oa, ob;
  oa.base = a; oa.dtype = d->dtype_a; oa.batch_stride = batch > 1 ? d->stride_a : 0;
  oa.mn_major = d->trans_a;
  oa.lines = d->trans_a ? d->k : d->m;
  oa.inner = d->trans_a ? d->m : d->k;
  oa.ld = d->lda ? d->lda : oa.inner;
  ob.base = b; ob.dtype = d->dtype_b; ob.batch_stride = batch > 1 ? d->stride_b : 0;
  ob.mn_major = !d->trans_b;
  ob.lines = d->trans_b ? d->n : d->k;
  ob.inner = d->trans_b ? d->k : d->n;
  ob.ld = d->ldb ? d->ldb : ob.inner;
  oa.outer = ob.outer = outer;
  oa.outer_stride = d->stride_a_outer;
  ob.outer_stride = d->stride_b_outer;
  if (oa.ld < oa.inner || ob.ld < ob.inner) return GB_ERR_INVALID;
  fill_dense_gather(p.ga, oa);
  fill_dense_gather(p.gbsrc, ob);
  p.a_mn_major = oa.mn_major;
  p.b_mn_major = ob.mn_major;

  const uint32_t out_inner = d->transpose_out ? d->m : d->n;
  const uint32_t ldc = d->ldc ? d->ldc : out_inner;
  if (ldc < out_inner) return GB_ERR_INVALID;
  set_output(p, c, d->dtype_c, ldc, batch > 1 ? d->stride_c : 0, d->transpose_out, d->accumulate, ep);

  const uint32_t min_bn = (plan.tensor && ob.mn_major) ? epl : 32;
  if (outer > 1 && !plan.tensor) return GB_ERR_UNSUPPORTED;
  if (outer > 1 && (d->stride_c_outer * elem_size(d->dtype_c)) % 16 != 0) p.vec_store = 0;   // per-lane stores reach any offset
  int rc = finish_plan(h, plan, outer == 1, min_bn, ep);   // no K split across two batch levels
  if (rc != GB_OK) return rc;
  if (plan.tensor) {
    p.a_kind = dense_tma(&plan.tmap_a, oa, smem_bf16, batch, 128, epl) ? (oa.mn_major ? gb::kDenseMN : gb::kDenseK) : gb::kGather;
    p.b_kind = dense_tma(&plan.tmap_b, ob, smem_bf16, batch, p.bn, epl) ? (ob.mn_major ? gb::kDenseMN : gb::kDenseK) : gb::kGather;
    if (outer > 1 && (p.a_kind == gb::kGather || p.b_kind == gb::kGather)) return GB_ERR_UNSUPPORTED;   // the gather warps know one batch stride
    CUtensorMap single = plan.tmap_b;
    if (!try_pair(h, plan, min_bn, [&](uint32_t rows) { return dense_tma(&plan.tmap_b, ob, smem_bf16, batch, rows, epl); }))
      plan.tmap_b = single;
  }
  return GB_OK;
}

// Everything a call decides before it launches: workspace use, the result's TMA map, stage count, what to launch.
// No CUDA launch happens here, so a prepared plan can be kept and launched again (the plan cache below).
int prepare_plan(const gb_handle* h, Plan& plan, void* workspace, size_t workspace_bytes) {
  GemmParams& p = plan.p;
  gb_plan_info& info = plan.info;
  info = gb_plan_info{};
  plan.reduce = false;
  if (p.m == 0 || p.n == 0 || p.batch == 0) {   // an empty grid is a no-op (src/gpu/gpu.zig:612)
    plan.launch = kLaunchNone;
    return GB_OK;
  }
  if (plan.direct) {
    plan.launch = kLaunchDirect;
    info.tensor_path = 0; info.a_kind = info.b_kind = (uint32_t)gb::kGather;
    info.tile_m = 128; info.tile_n = 32; info.stages = 1; info.splits = 1; info.k_blocks = 1;
    info.work_items = (p.m + 127) / 128; info.kernel_launches = 1;
    return GB_OK;
  }
  if (plan.direct_wgrad_blocks > 0 && workspace != nullptr && workspace_bytes >= plan.direct_wgrad_bytes && aligned16(workspace)) {
    plan.launch = kLaunchDirectWgrad;
    plan.reduce = true;
    p.partial = (float*)workspace;
    p.splits = plan.direct_wgrad_blocks;
    info.tensor_path = 0; info.a_kind = info.b_kind = (uint32_t)gb::kGather;
    info.tile_m = p.m; info.tile_n = p.n; info.stages = 1; info.splits = p.splits; info.k_blocks = 1;
    info.work_items = p.splits; info.kernel_launches = 2;
    return GB_OK;
  }
  if (p.splits > 1) {
    if (workspace == nullptr || workspace_bytes < plan.workspace || !aligned16(workspace)) {
      // Without room for partials the product runs unsplit rather than failing.
      p.splits = 1;
      p.k_blocks_per_split = p.k_blocks_total;
    } else {
      p.partial = (float*)workspace;
    }
  }
  p.spin_limit = knobs().test_spin_limit;
  info.tensor_path = plan.tensor;
  info.a_kind = plan.tensor ? p.a_kind : (uint32_t)gb::kGather;
  info.b_kind = plan.tensor ? p.b_kind : (uint32_t)gb::kGather;
  info.tile_m = plan.tensor ? (p.cta_pair ? 256 : 128) : 64;
  info.tile_n = p.bn;
  info.splits = p.splits;
  info.k_blocks = p.k_blocks_total;
  info.work_items = p.tiles_m * p.tiles_n * p.batch * p.splits;
  info.kernel_launches = p.k == 0 ? 1 : (p.splits > 1 ? 2 : 1);
  p.div_splits = gb::make_fastdiv_host(p.splits);
  p.div_per_batch = gb::make_fastdiv_host(p.tiles_m * p.tiles_n);
  p.div_band = gb::make_fastdiv_host(p.group_m * p.tiles_n);
  p.div_group = gb::make_fastdiv_host(p.group_m);
  // Row-major results whose rows start on 16-byte boundaries leave through a TMA store: a map of C as
  // {n, m, batch} with a box of 64 bytes x 32 rows, the block one epilogue warp stages per chunk.
  p.tma_store = 0;
  std::memset(&plan.tmap_c, 0, sizeof(plan.tmap_c));
  if (plan.tensor && p.k != 0 && p.splits > 1 && p.epi_groups == 2 && (p.n & 3) == 0 && !knobs().no_tma_store) {
    // K parts leave their partial tiles the same way, through a map of the partial buffer {n, m, split * batch}
    const uint64_t dims[3] = {p.n, p.m, (uint64_t)p.splits * p.batch};
    const uint64_t strides[2] = {(uint64_t)p.n * 4, (uint64_t)p.n * 4 * p.m};
    const uint32_t box[3] = {16, 32, 1};
    p.tma_store = encode_map(&plan.tmap_c, false, p.partial, 3, dims, strides, box, false, nullptr, true) ? 1 : 0;
  } else if (plan.tensor && p.k != 0 && p.splits == 1 && p.vec_store && !p.transpose_out && !p.rowmap.enabled && p.epi_groups == 2 &&
      !knobs().no_tma_store) {
    const uint32_t es = p.c_is_bf16 ? 2 : 4;
    if (p.batch_inner) {   // two batch levels: a four-dimensional map of C
      const uint64_t dims[4] = {p.n, p.m, p.batch_inner, p.batch / p.batch_inner};
      const uint64_t strides[3] = {(uint64_t)p.ldc * es, p.batch_inner > 1 ? p.stride_c * es : (uint64_t)p.ldc * es * p.m, p.stride_c_outer * es};
      const uint32_t box[4] = {64 / es, 32, 1, 1};
      p.tma_store = encode_map(&plan.tmap_c, p.c_is_bf16, p.c, 4, dims, strides, box, false, nullptr, true) ? 1 : 0;
    } else {
      const uint64_t dims[3] = {p.n, p.m, p.batch};
      const uint64_t strides[2] = {(uint64_t)p.ldc * es, p.batch > 1 ? p.stride_c * es : (uint64_t)p.ldc * es * p.m};
      const uint32_t box[3] = {64 / es, 32, 1};
      p.tma_store = encode_map(&plan.tmap_c, p.c_is_bf16, p.c, 3, dims, strides, box, false, nullptr, true) ? 1 : 0;
    }
    // 2: the chunk epilogue without run-time options (bf16 result = max(acc + bias, floor), nothing read back)
    if (p.tma_store && p.c_is_bf16 && !p.accumulate && !p.residual && !p.round_tf32 && !p.stats) p.tma_store = 2;
  }
  if (plan.tensor) {
    // The stage ring takes what the epilogue's own shared memory leaves of the 227 KB a CTA can have.
    const uint32_t b_lines = p.cta_pair ? p.bn / 2 : p.bn;
    const size_t stage = (p.a_stage_bytes ? p.a_stage_bytes : 128 * 128 * std::max(p.k_mul, 1u)) +
                         (size_t)std::max(p.col_taps, 1u) * b_lines * 128 * std::max(p.k_mul, 1u);
    const size_t fixed = gb::gemm_smem_bytes(p) - (size_t)p.stages * stage;
    const uint32_t fit = (uint32_t)((227 * 1024 - fixed) / stage);
    p.stages = std::max(2u, std::min(p.stages, fit));
  }
  info.stages = p.stages;
  if (p.stats) {
    if (!p.tma_store || p.k == 0 || p.splits != 1 || p.tiles_n != 1) return GB_ERR_UNSUPPORTED;
    p.stat_partial = nullptr;
    if (plan.stats_ordered) {
      // every CTA leaves its warps' partial sums in the workspace (8 KB each) for the ordered combine
      plan.stats_ctas = gb::gemm_grid_ctas(p, h->sm_count);
      const size_t need = (size_t)plan.stats_ctas * kStatsPartialBytesPerCta;
      if (workspace == nullptr || workspace_bytes < need || !aligned16(workspace)) return GB_ERR_WORKSPACE;
      p.stat_partial = (float*)workspace;
      info.kernel_launches += 1;
    }
  }
  if (p.k == 0) {
    // An empty contraction is a zero product: only the epilogue runs (through the reduce kernel, zero parts).
    p.splits = 0;
    p.partial = nullptr;
    plan.launch = kLaunchEmptyK;
    plan.reduce = true;
    return GB_OK;
  }
  plan.launch = plan.tensor ? kLaunchTensor : kLaunchF32;
  plan.reduce = p.splits > 1;
  return GB_OK;
}

// Launches a prepared plan on `stream`.
int launch_plan(gb_handle* h, cudaStream_t stream, const Plan& plan) {
  h->last_plan = plan.info;
  cudaError_t e = cudaSuccess;
  switch (plan.launch) {
    case kLaunchNone: return GB_OK;
    case kLaunchDirect: e = gb::launch_conv_direct(plan.p, h->sm_count, stream); break;
    case kLaunchDirectWgrad: e = gb::launch_conv_direct_wgrad(plan.p, plan.direct_wgrad_blocks, stream); break;
    case kLaunchEmptyK: break;
    case kLaunchF32: e = gb::launch_gemm_f32(plan.p, stream); break;
    case kLaunchTensor:
      if (!plan.p.cta_pair && h->test_drops_left > 0 && knobs().test_drop_kblock) {
        GemmParams injected = plan.p;   // host-requested failure injection (tests): this launch leaves out one K block's copies
        injected.test_drop_kblock = knobs().test_drop_kblock;
        --h->test_drops_left;
        e = gb::launch_gemm_sm100(injected, plan.tmap_a, plan.tmap_b, plan.tmap_c, h->sm_count, stream);
      } else {
        e = gb::launch_gemm_sm100(plan.p, plan.tmap_a, plan.tmap_b, plan.tmap_c, h->sm_count, stream);
      }
      break;
  }
  if (e == cudaSuccess && plan.reduce) e = gb::launch_splitk_reduce(plan.p, stream);
  if (e == cudaSuccess && plan.p.stats && plan.p.stat_partial != nullptr) e = gb::launch_stats_combine(plan.p, plan.stats_ctas, stream);
  return e == cudaSuccess ? GB_OK : cuda_fail(h, e);
}

int run_plan(gb_handle* h, cudaStream_t stream, Plan& plan, void* workspace, size_t workspace_bytes) {
  const int rc = prepare_plan(h, plan, workspace, workspace_bytes);
  return rc == GB_OK ? launch_plan(h, stream, plan) : rc;
}

// ---- plan cache -------------------------------------------------------------------------------------
// Planning a call costs the host ~15 us (the cost model and up to three cuTensorMapEncodeTiled calls), more than
// most ResNet layers take on the device, and a training step or an executor pass issues the same calls again and
// again.  A handle therefore keeps the prepared plans of its last calls, keyed by everything that went into them
// (descriptor, operand and result addresses, epilogue, workspace): a repeated call is a key compare and a launch.
// Tensor maps hold addresses and shapes only, so a cached plan stays valid whatever the buffers contain.
PlanKey make_key(uint32_t kind, const void* desc, size_t desc_bytes, const void* a, const void* b, const void* c, const gb_epilogue* ep,
                 const void* workspace, size_t workspace_bytes) {
  PlanKey key;
  std::memset(&key, 0, sizeof(key));
  key.kind = kind;
  std::memcpy(key.desc, desc, std::min(desc_bytes, sizeof(key.desc)));
  key.ptr[0] = (uint64_t)(uintptr_t)a; key.ptr[1] = (uint64_t)(uintptr_t)b; key.ptr[2] = (uint64_t)(uintptr_t)c;
  key.ptr[3] = (uint64_t)(uintptr_t)workspace; key.ptr[4] = (uint64_t)workspace_bytes;
  if (ep) {
    key.ptr[5] = (uint64_t)(uintptr_t)ep->bias; key.ptr[6] = (uint64_t)(uintptr_t)ep->residual;
    key.ptr[7] = ((uint64_t)(uint32_t)ep->activation << 32) | (uint32_t)ep->flags;
    if (ep->bn_stats) {
      key.ptr[8] = (uint64_t)(uintptr_t)ep->bn_stats->shift; key.ptr[9] = (uint64_t)(uintptr_t)ep->bn_stats->sums;
      key.ptr[10] = 1 + (uint64_t)ep->bn_stats->ordered;
    }
  }
  uint64_t hash = 1469598103934665603ull;
  const unsigned char* bytes = (const unsigned char*)&key;
  for (size_t i = 0; i < offsetof(PlanKey, hash); ++i) hash = (hash ^ bytes[i]) * 1099511628211ull;
  key.hash = hash;
  return key;
}

Plan* cache_find(gb_handle* h, const PlanKey& key) {
  if (knobs().no_plan_cache) return nullptr;
  for (CachedPlan& e : h->cache)
    if (e.key.hash == key.hash && std::memcmp(&e.key, &key, sizeof(key)) == 0) {
      e.stamp = ++h->cache_clock;
      ++h->cache_hits;
      return &e.plan;
    }
  return nullptr;
}

void cache_store(gb_handle* h, const PlanKey& key, const Plan& plan) {
  if (knobs().no_plan_cache) return;
  constexpr size_t kMaxPlans = 256;
  if (h->cache.size() < kMaxPlans) {
    h->cache.push_back(CachedPlan{key, plan, ++h->cache_clock});
    return;
  }
  CachedPlan* oldest = &h->cache[0];
  for (CachedPlan& e : h->cache)
    if (e.stamp < oldest->stamp) oldest = &e;
  *oldest = CachedPlan{key, plan, ++h->cache_clock};
}

// ---- convolution planning ---------------------------------------------------------------------------
int validate_conv(const gb_conv_desc* d) {
  if (!d) return GB_ERR_INVALID;
  const gb_conv_geometry& g = d->geo;
  if (g.n == 0 || g.h == 0 || g.w == 0 || g.c == 0 || g.k == 0 || g.stride == 0 || g.c_out == 0) return GB_ERR_INVALID;
  const uint32_t dil = g.dilation ? g.dilation : 1;
  if (dil * (g.k - 1) + 1 > g.h + 2 * g.pad || dil * (g.k - 1) + 1 > g.w + 2 * g.pad) return GB_ERR_INVALID;
  const uint32_t oh = (g.h + 2 * g.pad - dil * (g.k - 1) - 1) / g.stride + 1;   // src/gpu/math/conv.zig:24-30
  const uint32_t ow = (g.w + 2 * g.pad - dil * (g.k - 1) - 1) / g.stride + 1;
  if (g.out_h != oh || g.out_w != ow) return GB_ERR_INVALID;
  if ((uint64_t)g.positions != (uint64_t)g.n * oh * ow) return GB_ERR_INVALID;
  if (g.c_step != 0 && g.c_step < g.c) return GB_ERR_INVALID;
  if (d->groups > 1 && (g.c % d->groups != 0 || g.c_out % d->groups != 0)) return GB_ERR_INVALID;
  if (d->dtype_x > GB_BF16 || d->dtype_w > GB_BF16 || d->dtype_y > GB_BF16 || d->math > GB_MATH_BF16 || d->w_layout > 1) return GB_ERR_INVALID;
  return GB_OK;
}

gb::ConvGeo to_geo(const gb_conv_geometry& g, uint32_t y_step = 0, uint32_t w_step = 0) {
  gb::ConvGeo o;
  o.y_step = y_step ? y_step : g.c_out;
  o.w_step = w_step ? w_step : g.c_out;
  o.n = g.n; o.h = g.h; o.w = g.w; o.c = g.c; o.k = g.k; o.stride = g.stride; o.pad = g.pad;
  o.dilation = g.dilation ? g.dilation : 1;
  o.out_h = g.out_h; o.out_w = g.out_w; o.c_out = g.c_out;
  o.c_step = g.c_step ? g.c_step : g.c;
  return o;
}

// Splits `count` consecutive positions of a (grid_h x grid_w) grid into a box of whole rows (and whole
// images when count spans several).  False when the positions do not form such a box.
bool patch_box(uint32_t count, uint32_t grid_h, uint32_t grid_w, uint32_t& bw, uint32_t& bh, uint32_t& bn) {
  if (grid_w == 0 || count % grid_w != 0) return false;
  const uint32_t per_image = grid_h * grid_w;
  if (per_image % count == 0) {
    bw = grid_w; bh = count / grid_w; bn = 1;
  } else if (count % per_image == 0) {
    bw = grid_w; bh = grid_h; bn = count / per_image;
  } else {
    return false;
  }
  return bw <= 256 && bh <= 256 && bn <= 256;
}

// 4-D map over an NHWC tensor {channels, width, height, images} with a box of `epl` channels x (bw, bh, bn).
bool nhwc_tma(CUtensorMap* map, const void* base, bool smem_bf16, uint32_t dtype, uint32_t channels, uint32_t c_step, uint32_t width,
              uint32_t height, uint32_t images, uint32_t epl, uint32_t bw, uint32_t bh, uint32_t bn, bool mn_major = false,
              uint32_t conv_stride = 1, bool oob_nan = false) {
  const uint32_t es = smem_bf16 ? 2 : 4;
  if ((dtype == GB_BF16) != smem_bf16) return false;
  if (channels % epl != 0 || !aligned16(base) || ((uint64_t)c_step * es) % 16 != 0) return false;
  const uint64_t dims[4] = {channels, width, height, images};
  const uint64_t strides[3] = {(uint64_t)c_step * es, (uint64_t)c_step * es * width, (uint64_t)c_step * es * width * height};
  // A strided convolution visits every conv_stride-th column and row: the box spans bw*stride x bh*stride
  // input pixels and TMA's traversal stride keeps one in conv_stride of them, landing compact in shared memory.
  const uint32_t box[4] = {epl, bw * conv_stride, bh * conv_stride, bn};
  const uint32_t estr[4] = {1, conv_stride, conv_stride, 1};
  if (box[1] > 256 || box[2] > 256) return false;
  return encode_map(map, smem_bf16, base, 4, dims, strides, box, !smem_bf16 && mn_major, estr, false, oob_nan);
}

// K walk of the patch boxes of a forward pass (taps in storage order, patch origin at -pad).
void walk_forward(gb::TapWalk& wk, const gb::ConvGeo& g, uint32_t epl) {
  wk.cblocks = std::max(1u, g.c / epl); wk.n1 = g.k; wk.n2 = g.k;
  wk.grid_h = g.out_h; wk.grid_w = g.out_w;
  wk.div_image = gb::make_fastdiv_host(g.out_h * g.out_w); wk.div_w = gb::make_fastdiv_host(g.out_w);
  wk.row_scale = g.stride;
  wk.y0 = wk.z0 = -(int32_t)g.pad;
  wk.y_step = wk.z_step = (int32_t)g.dilation;
  wk.tap0 = 0; wk.tap_x = 1; wk.tap_y = (int32_t)g.k;
}

// K walk of a stride-1 input gradient: dy patches with mirrored tap offsets, filter taps in storage order.
void walk_dgrad_unit(gb::TapWalk& wk, const gb::ConvGeo& g, uint32_t epl) {
  wk.cblocks = std::max(1u, g.c_out / epl); wk.n1 = g.k; wk.n2 = g.k;
  wk.grid_h = g.h; wk.grid_w = g.w;
  wk.div_image = gb::make_fastdiv_host(g.h * g.w); wk.div_w = gb::make_fastdiv_host(g.w);
  wk.row_scale = 1;
  wk.y0 = wk.z0 = (int32_t)g.pad;
  wk.y_step = wk.z_step = -(int32_t)g.dilation;
  wk.tap0 = 0; wk.tap_x = 1; wk.tap_y = (int32_t)g.k;
}

// A strided 1x1 convolution without padding reads every s-th pixel of every s-th row and nothing else: the
// patch tensor is a VIEW of x with doubled (s-fold) pixel and row pitch.  Boxes of that view fetch only the
// pixels that are used; the traversal-stride boxes of `nhwc_tma` span all s*s of them (0.56 ms for the 64->192
// shortcut of a 4096-image ResNet pass, four times its useful bytes).
bool nhwc_view_tma(CUtensorMap* map, const void* base, bool smem_bf16, uint32_t dtype, const gb::ConvGeo& g, uint32_t epl, uint32_t bw,
                   uint32_t bh, uint32_t bn, bool mn_major) {
  const uint32_t es = smem_bf16 ? 2 : 4;
  if ((dtype == GB_BF16) != smem_bf16) return false;
  if (g.c % epl != 0 || !aligned16(base) || ((uint64_t)g.c_step * es) % 16 != 0) return false;
  const uint64_t dims[4] = {g.c, g.out_w, g.out_h, g.n};
  const uint64_t strides[3] = {(uint64_t)g.c_step * es * g.stride, (uint64_t)g.c_step * es * g.w * g.stride, (uint64_t)g.c_step * es * g.w * g.h};
  const uint32_t box[4] = {epl, bw, bh, bn};
  if (box[1] > 256 || box[2] > 256) return false;
  return encode_map(map, smem_bf16, base, 4, dims, strides, box, !smem_bf16 && mn_major);
}

// Switches a planned patch product to column-patch stages when its geometry allows: the tile is whole rows of
// one image, patch rows step one image row per output row, every operand arrives by TMA, K is not split, and
// a tap's row offset keeps the 1024-byte swizzle atoms of the A part aligned (box width x row step a multiple of
// eight lines).  One stage then serves all taps of a tap column: a third as many stages, barrier round trips
// and producer iterations per tile for a 3x3 filter, and (box_h + 2) / (3 * box_h) of the activation bytes.
// `encode_a(rows)` re-encodes the activation map for a box of `rows` image rows.
// `min_fit`: stages that must fit (three by default: with two the ring holds less than a tile).
template <class EncodeA>
void try_column_stages(Plan& plan, EncodeA encode_a, uint32_t min_fit = 3) {
  GemmParams& p = plan.p;
  if (knobs().no_column_stages || min_fit == 0) return;
  const gb::TapWalk& wk = p.walk;
  if (!plan.tensor || p.a_kind != gb::kPatchK || p.b_kind == gb::kGather || p.splits != 1 || p.box_n != 1 || p.bn > 256) return;
  if (wk.n2 < 2 || wk.n2 > 7 || wk.row_scale != 1 || wk.z_step == 0) return;
  const uint32_t row_step = (uint32_t)std::abs(wk.z_step), epl = p.tf32 ? 32 : 64;
  if ((p.box_w * row_step) % 8 != 0) return;
  const uint32_t rows = p.box_h + (wk.n2 - 1) * row_step;
  if (rows > 256) return;
  const uint32_t b_lines = p.cta_pair ? p.bn / 2 : p.bn;
  const uint32_t boxes_b = (p.b_kind == gb::kDenseMN ? b_lines / epl : 1u) * wk.n2;
  if (1 + boxes_b > 32) return;
  const uint32_t a_box = rows * p.box_w * 128, a_stage = (a_box + 1023) & ~1023u;
  const size_t stage = a_stage + (size_t)wk.n2 * b_lines * 128;
  const size_t room = 227 * 1024 - 2048 - gb::kStoreSmemBytes - (p.stats ? 8 * gb::kStatBytesPerWarp : 0);
  if (room / stage < min_fit) return;
  if (!encode_a(rows)) return;
  p.col_taps = wk.n2;
  p.a_stage_bytes = a_stage;
  p.a_box_bytes = a_box;
  p.col_a_step16 = wk.z_step * (int32_t)(p.box_w * 8);
  p.col_a_first16 = wk.z_step < 0 ? (int32_t)((wk.n2 - 1) * row_step * p.box_w * 8) : 0;
  p.k_blocks_total = wk.n1 * wk.cblocks;
  p.k_blocks_per_split = p.k_blocks_total;
  p.stages = (uint32_t)std::min<size_t>(8, room / stage);
}

int plan_conv(const gb_handle* h, int pass, const gb_conv_desc* d, const void* act, const void* other, void* out,
              const gb_epilogue* ep, Plan& plan, const gb_dx_stats* dxs = nullptr, const uint16_t* affine_scale = nullptr,
              const uint16_t* affine_shift = nullptr, uint32_t y_step = 0, uint32_t w_step = 0) {
  std::memset(&plan.p, 0, sizeof(plan.p));
  GemmParams& p = plan.p;
  p.affine_scale = affine_scale;
  p.affine_shift = affine_shift;
  const bool affine = affine_scale != nullptr;   // the patch operand is transformed while it is gathered: no TMA, no FMA kernel
  if (affine && (d->dtype_x != GB_BF16 || (d->math != GB_MATH_BF16 && d->math != GB_MATH_F32) || pass == 1)) return GB_ERR_UNSUPPORTED;
  const gb::ConvGeo g = to_geo(d->geo, y_step, w_step);
  p.geo = g;
  p.batch = 1;
  uint32_t math = d->math;
  if (math == GB_MATH_F32 && (d->dtype_x == GB_BF16 || d->dtype_y == GB_BF16)) math = GB_MATH_BF16;
  plan.tensor = math != GB_MATH_F32;
  p.tf32 = math == GB_MATH_TF32;
  const bool smem_bf16 = math == GB_MATH_BF16;
  const uint32_t epl = p.tf32 ? 32 : 64;
  const uint32_t taps = g.k * g.k;
  const uint32_t positions = d->geo.positions;
  if ((g.y_step != g.c_out || g.w_step != g.c_out) && (d->w_layout != 0 || dxs || (ep && ep->bn_stats))) return GB_ERR_UNSUPPORTED;   // group slices: plain layers only
  const uint32_t pixels = g.n * g.h * g.w;
  uint32_t min_bn = 32;
  // A pass with statistics stores the very bits of the plain pass (tests/gpu.zig:205), so it has to add up K in the same
  // order: column-patch stages walk the taps column by column, the plain walk row by row.  The plain pass is planned first
  // and the statistics plan (one column tile, more shared memory: possibly another tile width or CTA mode) follows its choice.
  int want_cols = -1;
  if ((ep && ep->bn_stats) || dxs) {
    Plan plain;
    gb_epilogue bare = ep ? *ep : gb_epilogue{};
    bare.bn_stats = nullptr;
    const int rc = plan_conv(h, pass, d, act, other, out, ep ? &bare : nullptr, plain, nullptr, affine_scale, affine_shift, y_step, w_step);
    if (rc != GB_OK) return rc;
    want_cols = plain.p.col_taps != 0 ? 1 : 0;
  }

  if (pass == 0) {
    // y[positions, c_out] = patches(x)[positions, taps*c] * w[taps*c, c_out]
    p.m = positions; p.n = g.c_out; p.k = taps * g.c;
    p.ga.base = act; p.ga.source = gb::kSrcPatch; p.ga.src_is_bf16 = d->dtype_x == GB_BF16;
    p.ga.lines_total = positions; p.ga.inner_total = p.k; p.ga.mn_major = 0;
    // Filters as grad stores them, (K, c_out), are an MN-major B; the prepared (c_out, K) copy is a K-major B.
    const bool w_rows = d->w_layout == 1;
    DenseOperand ob = w_rows ? DenseOperand{other, d->dtype_w, g.c_out, p.k, p.k, 0, false} : DenseOperand{other, d->dtype_w, p.k, g.c_out, g.w_step, 0, true};
    fill_dense_gather(p.gbsrc, ob);
    p.a_mn_major = 0; p.b_mn_major = w_rows ? 0 : 1;
    min_bn = (plan.tensor && !w_rows) ? epl : 32;
    set_output(p, out, d->dtype_y, g.y_step, 0, false, d->accumulate, ep);
    int rc = finish_plan(h, plan, true, min_bn, ep);
    if (rc != GB_OK) return rc;
    // A 3-channel 3x3 stride-1 layer over a bf16 map goes through the tensor kernel: its gather warps have a line builder
    // for exactly that window (13.6 against 29.9 us at batch 128, 378 against 605 us at batch 4096 for the FMA kernel).
    const bool stem_lines = smem_bf16 && d->dtype_x == GB_BF16 && g.c == 3 && g.c_step == 3 && g.k == 3 && g.stride == 1 && g.dilation == 1 &&
                            !w_rows && !knobs().no_stem_lines;   // (a prepared filter row of 27 values is no TMA operand)
    if (plan.tensor && gb::conv_direct_applies(p) && !knobs().no_direct_conv && !p.stats && !affine && !stem_lines) {
      plan.direct = true;
      plan.workspace = 0;
      return GB_OK;
    }
    if (plan.tensor) {
      p.a_kind = gb::kGather;
      walk_forward(p.walk, g, epl);
      const bool view = g.k == 1 && g.pad == 0 && g.stride > 1 && !knobs().no_strided_tma;
      if (affine) {
        // The virtual normalised input: fetched by TMA with NaN outside the image and rewritten in place by the transform
        // warps; where no TMA map fits it stays with the gather warps, which transform while they build the tile.
        if (smem_bf16 && g.c <= gb::kMaxXformTableChannels && patch_box(128, g.out_h, g.out_w, p.box_w, p.box_h, p.box_n) &&
            nhwc_tma(&plan.tmap_a, act, smem_bf16, d->dtype_x, g.c, g.c_step, g.w, g.h, g.n, epl, p.box_w, p.box_h, p.box_n, false, g.stride, true)) {
          p.a_kind = gb::kPatchK;
          p.xform = 1;
        }
      } else if (view && patch_box(128, g.out_h, g.out_w, p.box_w, p.box_h, p.box_n) &&
          nhwc_view_tma(&plan.tmap_a, act, smem_bf16, d->dtype_x, g, epl, p.box_w, p.box_h, p.box_n, false)) {
        p.a_kind = gb::kPatchK;
        p.walk.row_scale = 1;   // rows of the view, not of x
      } else if ((g.stride == 1 || !knobs().no_strided_tma) && patch_box(128, g.out_h, g.out_w, p.box_w, p.box_h, p.box_n) &&
                 nhwc_tma(&plan.tmap_a, act, smem_bf16, d->dtype_x, g.c, g.c_step, g.w, g.h, g.n, epl, p.box_w, p.box_h, p.box_n, false, g.stride))
        p.a_kind = gb::kPatchK;
      p.b_kind = dense_tma(&plan.tmap_b, ob, smem_bf16, 1, p.bn, epl) ? (w_rows ? gb::kDenseK : gb::kDenseMN) : gb::kGather;
      const Plan before = plan;   // the CTA mode and the staging are chosen below, twice for a statistics plan that has to follow the plain one
      auto choose = [&](int pair_mode, uint32_t min_fit) {
        plan = before;
        CUtensorMap single = plan.tmap_b;
        // (the transform warps exist in the single-CTA kernel only)
        if (!try_pair(h, plan, min_bn, [&](uint32_t rows) { return dense_tma(&plan.tmap_b, ob, smem_bf16, 1, rows, epl); }, p.xform ? 2 : pair_mode))
          plan.tmap_b = single;
        if (g.stride == 1)
          try_column_stages(plan, [&](uint32_t rows) {
            return nhwc_tma(&plan.tmap_a, act, smem_bf16, d->dtype_x, g.c, g.c_step, g.w, g.h, g.n, epl, p.box_w, rows, 1, false, 1, p.xform != 0);
          }, min_fit);
      };
      if (want_cols < 0) {
        choose(0, 3);
      } else {
        choose(0, want_cols ? 2 : 0);
        if ((p.col_taps != 0) != (want_cols != 0)) choose(p.cta_pair ? 2 : 1, want_cols ? 2 : 0);
        if ((p.col_taps != 0) != (want_cols != 0)) return GB_ERR_UNSUPPORTED;
      }
    }
  } else if (pass == 1) {
    // dx[pixels, c] = patchesT(dy)[pixels, taps*c_out] * wT[taps*c_out, c]
    p.m = pixels; p.n = g.c; p.k = taps * g.c_out;
    p.dgrad = 1;
    p.ga.base = act; p.ga.source = gb::kSrcPatchT; p.ga.src_is_bf16 = d->dtype_y == GB_BF16;
    p.ga.lines_total = pixels; p.ga.inner_total = p.k; p.ga.mn_major = 0;
    p.gbsrc.base = other; p.gbsrc.source = gb::kSrcWeightT; p.gbsrc.src_is_bf16 = d->dtype_w == GB_BF16;
    p.gbsrc.lines_total = g.c; p.gbsrc.inner_total = p.k; p.gbsrc.mn_major = 0;
    p.a_mn_major = 0; p.b_mn_major = 0;
    set_output(p, out, d->dtype_x, g.c_step, 0, false, d->accumulate, nullptr);
    gb_bn_stats as_forward = {};
    gb_epilogue stats_ep = {};
    if (dxs) {
      // the backward sums ride on the machinery of the forward statistics: same shape limits, same per-warp sums
      if (!dxs->x || !dxs->mean || !dxs->inv_std || !dxs->gamma || !dxs->beta || !dxs->sums || d->dtype_x != GB_BF16 || d->accumulate ||
          g.stride != 1 || g.c_step != g.c || !aligned16(dxs->x))
        return GB_ERR_UNSUPPORTED;
      as_forward.shift = dxs->mean; as_forward.sums = dxs->sums; as_forward.ordered = dxs->ordered;
      stats_ep.bn_stats = &as_forward;
    }
    int rc = finish_plan(h, plan, true, 32, dxs ? &stats_ep : nullptr);
    if (rc != GB_OK) return rc;
    if (dxs) {
      p.stats = 2;
      p.stat_x = dxs->x; p.stat_inv_std = dxs->inv_std; p.stat_gamma = dxs->gamma; p.stat_beta = dxs->beta;
    }
    if (plan.tensor) {
      p.a_kind = gb::kGather;
      walk_dgrad_unit(p.walk, g, epl);
      if (g.stride == 1 && patch_box(128, g.h, g.w, p.box_w, p.box_h, p.box_n) &&
          nhwc_tma(&plan.tmap_a, act, smem_bf16, d->dtype_y, g.c_out, g.y_step, g.out_w, g.out_h, g.n, epl, p.box_w, p.box_h, p.box_n))
        p.a_kind = gb::kPatchK;
      p.b_kind = gb::kGather;
      const uint32_t es = smem_bf16 ? 2 : 4;
      if ((d->dtype_w == GB_BF16) == smem_bf16 && g.c_out % epl == 0 && aligned16(other) && p.bn <= 256) {
        const uint64_t dims[4] = {g.c_out, g.c, taps, 1};
        const uint64_t strides[3] = {(uint64_t)g.w_step * es, (uint64_t)g.w_step * es * g.c, (uint64_t)g.w_step * es * g.c * taps};
        const uint32_t box[4] = {epl, p.bn, 1, 1};
        if (((uint64_t)g.w_step * es) % 16 == 0 && encode_map(&plan.tmap_b, smem_bf16, other, 4, dims, strides, box)) p.b_kind = gb::kWeightK;
        const Plan before = plan;
        auto choose = [&](int pair_mode, uint32_t min_fit) {
          plan = before;
          CUtensorMap single = plan.tmap_b;
          if (!try_pair(h, plan, 32, [&](uint32_t rows) {
                const uint32_t half_box[4] = {epl, rows, 1, 1};
                return encode_map(&plan.tmap_b, smem_bf16, other, 4, dims, strides, half_box);
              }, pair_mode))
            plan.tmap_b = single;
          try_column_stages(plan, [&](uint32_t rows) {
            return nhwc_tma(&plan.tmap_a, act, smem_bf16, d->dtype_y, g.c_out, g.y_step, g.out_w, g.out_h, g.n, epl, p.box_w, rows, 1);
          }, min_fit);
        };
        if (want_cols < 0) {
          choose(0, 3);
        } else {
          choose(0, want_cols ? 2 : 0);
          if ((p.col_taps != 0) != (want_cols != 0)) choose(p.cta_pair ? 2 : 1, want_cols ? 2 : 0);
          if ((p.col_taps != 0) != (want_cols != 0)) return GB_ERR_UNSUPPORTED;
        }
      }
    }
  } else {
    // dw[taps*c, c_out] += patches(x)^T[taps*c, positions] * dy[positions, c_out]
    p.m = taps * g.c; p.n = g.c_out; p.k = positions;
    p.ga.base = other; p.ga.source = gb::kSrcPatch; p.ga.src_is_bf16 = d->dtype_x == GB_BF16;
    p.ga.lines_total = positions; p.ga.inner_total = p.m; p.ga.mn_major = 1;
    DenseOperand ob{act, d->dtype_y, positions, g.c_out, g.y_step, 0, true};
    fill_dense_gather(p.gbsrc, ob);
    p.a_mn_major = 1; p.b_mn_major = 1;
    min_bn = plan.tensor ? epl : 32;
    set_output(p, out, d->dtype_w, g.w_step, 0, false, d->accumulate, nullptr);
    int rc = finish_plan(h, plan, true, min_bn, nullptr);
    if (rc != GB_OK) return rc;
    // (the 3-channel bf16 stem: the tensor kernel's gather warps build its window lines, see the forward pass)
    const bool stem_lines = smem_bf16 && d->dtype_x == GB_BF16 && g.c == 3 && g.c_step == 3 && g.k == 3 && g.stride == 1 && g.dilation == 1 &&
                            !affine && !knobs().no_stem_lines;
    if (plan.tensor && gb::conv_direct_wgrad_applies(p) && !knobs().no_direct_conv && !affine && !stem_lines) {
      plan.direct_wgrad_blocks = gb::conv_direct_wgrad_blocks(p, h->sm_count);
      plan.direct_wgrad_bytes = (size_t)plan.direct_wgrad_blocks * p.m * p.n * sizeof(float);
    }
    if (plan.tensor) {
      p.a_kind = gb::kGather;
      p.walk.div_image = gb::make_fastdiv_host(g.out_h * g.out_w);   // the stem lines split a position with these
      p.walk.div_w = gb::make_fastdiv_host(g.out_w);
      const bool view = g.k == 1 && g.pad == 0 && g.stride > 1 && !knobs().no_strided_tma;
      if (affine) {
        // as in the forward pass: TMA with NaN outside the image + the transform warps, else the gather warps
        if (smem_bf16 && g.c <= gb::kMaxXformTableChannels && patch_box(epl, g.out_h, g.out_w, p.box_w, p.box_h, p.box_n) &&
            nhwc_tma(&plan.tmap_a, other, smem_bf16, d->dtype_x, g.c, g.c_step, g.w, g.h, g.n, epl, p.box_w, p.box_h, p.box_n, true, g.stride, true)) {
          p.a_kind = gb::kPatchMN;
          p.xform = 1;
        }
      } else if (view && patch_box(epl, g.out_h, g.out_w, p.box_w, p.box_h, p.box_n) &&
          nhwc_view_tma(&plan.tmap_a, other, smem_bf16, d->dtype_x, g, epl, p.box_w, p.box_h, p.box_n, true)) {
        p.a_kind = gb::kPatchMN;
        p.patch_view = 1;
      } else if ((g.stride == 1 || !knobs().no_strided_tma) && patch_box(epl, g.out_h, g.out_w, p.box_w, p.box_h, p.box_n) &&
                 nhwc_tma(&plan.tmap_a, other, smem_bf16, d->dtype_x, g.c, g.c_step, g.w, g.h, g.n, epl, p.box_w, p.box_h, p.box_n, true, g.stride))
        p.a_kind = gb::kPatchMN;
      p.b_kind = dense_tma(&plan.tmap_b, ob, smem_bf16, 1, p.bn, epl) ? gb::kDenseMN : gb::kGather;
      {
        CUtensorMap single = plan.tmap_b;
        if (!try_pair(h, plan, min_bn, [&](uint32_t rows) { return dense_tma(&plan.tmap_b, ob, smem_bf16, 1, rows, epl); }, p.xform ? 2 : 0, true))
          plan.tmap_b = single;
      }
      // Both operands are MN-major (one line per position), so two K blocks per stage are simply boxes of twice
      // as many lines: half the stages, barrier round trips and producer iterations for the same MMAs.  (The K
      // loop of a weight gradient is producer-bound: ~570 cycles per stage against 256 of MMA time.)
      uint32_t bw2, bh2, bn2;
      CUtensorMap a2, b2;
      if (!p.cta_pair && p.a_kind == gb::kPatchMN && p.b_kind == gb::kDenseMN && !knobs().no_wide_stages && p.k_blocks_total >= 8 &&
          patch_box(2 * epl, g.out_h, g.out_w, bw2, bh2, bn2) &&
          (p.patch_view ? nhwc_view_tma(&a2, other, smem_bf16, d->dtype_x, g, epl, bw2, bh2, bn2, true)
                        : nhwc_tma(&a2, other, smem_bf16, d->dtype_x, g.c, g.c_step, g.w, g.h, g.n, epl, bw2, bh2, bn2, true, g.stride, p.xform != 0)) &&
          (227 * 1024 - 2048 - gb::kStoreSmemBytes) / (2 * (128 * 128 + p.bn * 128)) >= 3 &&   // two-block stages only while three of them fit
          dense_tma(&b2, ob, smem_bf16, 1, p.bn, epl, 2)) {
        plan.tmap_a = a2; plan.tmap_b = b2;
        p.box_w = bw2; p.box_h = bh2; p.box_n = bn2;
        p.k_mul = 2;
        p.k_blocks_total = ceil_div(p.k_blocks_total, 2);
        p.k_blocks_per_split = std::max(1u, ceil_div(p.k_blocks_total, p.splits));
        p.splits = std::max(1u, ceil_div(p.k_blocks_total, p.k_blocks_per_split));
        plan.workspace = p.splits > 1 ? (size_t)p.splits * p.batch * p.m * p.n * sizeof(float) : 0;
        p.stages = std::min<uint32_t>(8, (227 * 1024 - 2048) / (2 * (128 * 128 + p.bn * 128)));
      }
    }
    plan.workspace = std::max(plan.workspace, plan.direct_wgrad_bytes);
  }
  return GB_OK;
}

// bf16 math over f32 master filters (the reference packs them to bf16 on every call: `packMatrix` in
// `convImplicitForward`, src/gpu/gpu.zig:926-960).  Read as f32 they could only be gathered -- 185 us instead of
// 27 us for a 64-channel layer -- so the forward pass and the input gradient first round them into the head of
// the caller's workspace (one cast launch over a few hundred KB) and then run as if bf16 filters had been
// passed.  Without a workspace that large the gathered plan runs as before.
bool wants_filter_shadow(const gb_conv_desc* d) {
  uint32_t math = d->math;
  if (math == GB_MATH_F32 && (d->dtype_x == GB_BF16 || d->dtype_y == GB_BF16)) math = GB_MATH_BF16;
  return math == GB_MATH_BF16 && d->dtype_w == GB_F32;
}
size_t filter_shadow_bytes(const gb_conv_desc* d) {
  const size_t elems = (size_t)d->geo.k * d->geo.k * (d->geo.c / std::max<uint32_t>(d->groups, 1)) * d->geo.c_out;
  return (elems * 2 + 255) & ~(size_t)255;
}
// Returns the descriptor / filter pointer / workspace to continue with; `shadow` receives the patched descriptor.
int make_filter_shadow(gb_handle* h, cudaStream_t stream, const gb_conv_desc*& desc, gb_conv_desc& shadow, const void*& w, void*& workspace,
                       size_t& workspace_bytes) {
  if (!wants_filter_shadow(desc)) return GB_OK;
  const size_t need = filter_shadow_bytes(desc);
  if (workspace == nullptr || workspace_bytes < need || !aligned16(workspace)) return GB_OK;
  const size_t elems = (size_t)desc->geo.k * desc->geo.k * (desc->geo.c / std::max<uint32_t>(desc->groups, 1)) * desc->geo.c_out;
  const int rc = gb_cast(stream, GB_F32, GB_BF16, w, workspace, elems);
  if (rc != GB_OK) return rc == GB_ERR_CUDA ? cuda_fail(h, cudaGetLastError()) : rc;
  shadow = *desc;
  shadow.dtype_w = GB_BF16;
  desc = &shadow;
  w = workspace;
  workspace = (char*)workspace + need;
  workspace_bytes -= need;
  return GB_OK;
}

// Input gradient of a strided convolution as up to stride^2 products, one per parity class of input pixels.
// Pixel (s*i + py, s*j + px) only receives taps ky with (py + pad - ky*dil) divisible by s (likewise kx), and
// through such a tap it reads dy at (i + (py + pad - ky*dil)/s, j + ...): a stride-1 walk over dy.  So each
// class is an ordinary patch product over its own taps -- TMA boxes of dy, filter taps through the
// {c_out, c_in, taps} map, 1/s^2 of the dense work, no multiplication by inserted zeros -- whose rows land on
// every s-th pixel of dx (`RowMap`).  Returns GB_ERR_UNSUPPORTED, with nothing launched, when a class
// cannot be fetched this way; the caller then takes the single gathered product.
int run_dgrad_classes(gb_handle* h, cudaStream_t stream, const gb_conv_desc* d, const void* dy, const void* w, void* dx) {
  const gb::ConvGeo g = to_geo(d->geo);
  const uint32_t s = g.stride, dil = g.dilation;
  uint32_t math = d->math;
  if (math == GB_MATH_F32 && (d->dtype_x == GB_BF16 || d->dtype_y == GB_BF16)) math = GB_MATH_BF16;
  if (math == GB_MATH_F32 || s < 2 || s > 4 || knobs().no_dgrad_classes) return GB_ERR_UNSUPPORTED;
  const bool tf32 = math == GB_MATH_TF32, smem_bf16 = !tf32;
  const uint32_t epl = tf32 ? 32 : 64, es = smem_bf16 ? 2 : 4;
  if ((d->dtype_y == GB_BF16) != smem_bf16 || (d->dtype_w == GB_BF16) != smem_bf16) return GB_ERR_UNSUPPORTED;
  if (g.c_out % epl != 0 || !aligned16(dy) || !aligned16(w)) return GB_ERR_UNSUPPORTED;
  uint32_t gcd = s, t = dil;
  while (t) { const uint32_t r = gcd % t; gcd = t; t = r; }
  const uint32_t tk = s / gcd;                       // taps of one class are tk apart
  struct Axis { uint32_t count, taps, k0; int32_t off0; };
  auto axis = [&](uint32_t len, uint32_t r) {
    Axis a{len > r ? (len - r + s - 1) / s : 0u, 0u, 0u, 0};
    for (uint32_t kk = 0; kk < g.k; ++kk) {
      const int32_t v = (int32_t)(r + g.pad) - (int32_t)(kk * dil);
      if (((v % (int32_t)s) + (int32_t)s) % (int32_t)s == 0) {
        a.k0 = kk; a.off0 = v / (int32_t)s; a.taps = (g.k - 1 - kk) / tk + 1;
        break;
      }
    }
    return a;
  };
  std::vector<Plan> plans;
  bool any_empty = false;
  const uint32_t taps = g.k * g.k;
  for (uint32_t py = 0; py < s; ++py)
    for (uint32_t px = 0; px < s; ++px) {
      const Axis ay = axis(g.h, py), ax = axis(g.w, px);
      if (ay.count == 0 || ax.count == 0) continue;
      if (ay.taps == 0 || ax.taps == 0) { any_empty = true; continue; }
      plans.emplace_back();
      Plan& plan = plans.back();
      std::memset(&plan.p, 0, sizeof(plan.p));
      GemmParams& p = plan.p;
      p.geo = g; p.batch = 1; p.dgrad = 1; p.tf32 = tf32;
      plan.tensor = true;
      p.m = g.n * ay.count * ax.count; p.n = g.c; p.k = ay.taps * ax.taps * g.c_out;
      set_output(p, dx, d->dtype_x, g.c_step, 0, false, d->accumulate, nullptr);
      if (finish_plan(h, plan, false, 32, nullptr) != GB_OK) return GB_ERR_UNSUPPORTED;
      if (!patch_box(128, ay.count, ax.count, p.box_w, p.box_h, p.box_n) ||
          !nhwc_tma(&plan.tmap_a, dy, smem_bf16, d->dtype_y, g.c_out, g.c_out, g.out_w, g.out_h, g.n, epl, p.box_w, p.box_h, p.box_n))
        return GB_ERR_UNSUPPORTED;
      p.a_kind = gb::kPatchK;
      const uint64_t dims[4] = {g.c_out, g.c, taps, 1};
      const uint64_t strides[3] = {(uint64_t)g.c_out * es, (uint64_t)g.c_out * es * g.c, (uint64_t)g.c_out * es * g.c * taps};
      const uint32_t box[4] = {epl, p.bn, 1, 1};
      if (p.bn > 256 || !encode_map(&plan.tmap_b, smem_bf16, w, 4, dims, strides, box)) return GB_ERR_UNSUPPORTED;
      p.b_kind = gb::kWeightK;
      CUtensorMap single = plan.tmap_b;
      if (!try_pair(h, plan, 32, [&](uint32_t rows) {
            const uint32_t half_box[4] = {epl, rows, 1, 1};
            return encode_map(&plan.tmap_b, smem_bf16, w, 4, dims, strides, half_box);
          }))
        plan.tmap_b = single;
      gb::TapWalk& wk = p.walk;
      wk.cblocks = g.c_out / epl; wk.n1 = ax.taps; wk.n2 = ay.taps;
      wk.grid_h = ay.count; wk.grid_w = ax.count;
      wk.div_image = gb::make_fastdiv_host(ay.count * ax.count); wk.div_w = gb::make_fastdiv_host(ax.count);
      wk.row_scale = 1;
      wk.y0 = ax.off0; wk.z0 = ay.off0;
      wk.y_step = wk.z_step = -(int32_t)(dil * tk / s);
      wk.tap0 = (int32_t)(ay.k0 * g.k + ax.k0); wk.tap_x = (int32_t)tk; wk.tap_y = (int32_t)(tk * g.k);
      gb::RowMap& rm = p.rowmap;
      rm.enabled = 1;
      rm.per_image = wk.div_image; rm.grid_w = wk.div_w;
      rm.h = g.h; rm.w = g.w; rm.scale = s; rm.off_y = py; rm.off_x = px;
    }
  // A 1x1 layer has ONE class with taps; where the image is whole blocks of s x s pixels its epilogue writes the other
  // pixels' zeros itself (each of its rows owns the block at its pixel), else dx is cleared in front.
  bool fill_in_kernel = false;
  if (any_empty && !d->accumulate && plans.size() == 1) {
    GemmParams& p = plans[0].p;
    fill_in_kernel = g.h % s == 0 && g.w % s == 0 && p.rowmap.off_y == 0 && p.rowmap.off_x == 0 && p.vec_store && p.n % 32 == 0 &&
                     !p.transpose_out && p.splits <= 1;
    if (fill_in_kernel) p.zero_fill = s;
  }
  if (any_empty && !d->accumulate && !fill_in_kernel) {
    // Pixels of a class without taps get no product; they are zero.  Only a dense dx can be cleared as a block.
    if (g.c_step != g.c) return GB_ERR_UNSUPPORTED;
    const cudaError_t e = cudaMemsetAsync(dx, 0, (size_t)g.n * g.h * g.w * g.c * elem_size(d->dtype_x), stream);
    if (e != cudaSuccess) return cuda_fail(h, e);
  }
  // Classes that agree on tile shape, pair mode and patch box run as ONE launch: the class is the batch index of
  // the work decode, and its tap walk, row map, row count and K length sit in a slot of the parameters.  (Four
  // launches of a strided ResNet layer cost ~13 us each, mostly fixed cost.)
  if (plans.size() >= 2 && plans.size() <= gb::kMaxClasses && !knobs().no_fused_classes) {
    size_t lead = 0;
    bool same = true;
    for (size_t i = 0; i < plans.size(); ++i) {
      const GemmParams &a = plans[i].p, &b = plans[0].p;
      same = same && a.bn == b.bn && a.cta_pair == b.cta_pair && a.box_w == b.box_w && a.box_h == b.box_h && a.box_n == b.box_n &&
             a.walk.grid_h == b.walk.grid_h && a.walk.grid_w == b.walk.grid_w && a.splits == 1 && a.col_taps == 0 && a.k_mul <= 1;
      if (a.k_blocks_total > plans[lead].p.k_blocks_total) lead = i;
    }
    if (same) {
      Plan fused = plans[lead];
      GemmParams& f = fused.p;
      f.n_classes = (uint32_t)plans.size();
      f.batch = f.n_classes;
      f.stride_c = 0;
      for (size_t i = 0; i < plans.size(); ++i) {
        const GemmParams& c = plans[i].p;
        f.cls[i].walk = c.walk; f.cls[i].rowmap = c.rowmap; f.cls[i].m = c.m; f.cls[i].k_blocks = c.k_blocks_total;
        f.m = std::max(f.m, c.m);
        f.tiles_m = std::max(f.tiles_m, c.tiles_m);
      }
      f.k_blocks_per_split = f.k_blocks_total;
      return run_plan(h, stream, fused, nullptr, 0);
    }
  }
  uint32_t launches = 0, items = 0;
  for (Plan& plan : plans) {
    const int rc = run_plan(h, stream, plan, nullptr, 0);
    if (rc != GB_OK) return rc;
    launches += h->last_plan.kernel_launches;
    items += h->last_plan.work_items;
  }
  h->last_plan.kernel_launches = launches;
  h->last_plan.work_items = items;
  return GB_OK;
}

// A grouped convolution as one product per group: group g reads input channels [g*cg, (g+1)*cg) of x (a channel slice:
// same pixel pitch), columns [g*og, (g+1)*og) of w and of y / dy (column slices: same row pitch), the way grad's
// `grouped_implicit` path launches its kernel once per group with `c_pitch` / `c_offset` (src/autograd/autograd.zig:1041-1050,
// src/gpu/args.zig:72).  `act`, `other`, `out` are the pass's operands in the order of plan_conv.
int run_grouped(gb_handle* h, cudaStream_t stream, int pass, const gb_conv_desc* desc, const void* act, const void* other, void* out,
                const gb_epilogue* ep, void* workspace, size_t workspace_bytes) {
  if (desc->w_layout != 0 || (ep && ep->bn_stats)) return GB_ERR_UNSUPPORTED;
  const uint32_t groups = desc->groups, cg = desc->geo.c / groups, og = desc->geo.c_out / groups;
  const uint32_t c_total = desc->geo.c_step ? desc->geo.c_step : desc->geo.c, o_total = desc->geo.c_out;
  const void* w = pass == 2 ? nullptr : other;
  gb_conv_desc whole = *desc;
  const gb_conv_desc* cast_desc = desc;
  uint32_t extra = 0;
  if (pass != 2) {
    const int rc = make_filter_shadow(h, stream, cast_desc, whole, w, workspace, workspace_bytes);   // the whole filter bank, once
    if (rc != GB_OK) return rc;
    extra = cast_desc == &whole ? 1u : 0u;
  }
  gb_conv_desc one = *cast_desc;
  one.groups = 1;
  one.geo.c = cg;
  one.geo.c_step = c_total;
  one.geo.c_out = og;
  const size_t es_x = elem_size(one.dtype_x), es_w = elem_size(one.dtype_w), es_y = elem_size(one.dtype_y);
  uint32_t launches = 0, items = 0;
  for (uint32_t g = 0; g < groups; ++g) {
    // which operand is what, per pass: fprop (x, w, y); dgrad (dy, w, dx); wgrad (dy, x, dw)
    const char* a = (const char*)act + (size_t)g * (pass == 0 ? cg * es_x : og * es_y);
    const char* b = pass == 2 ? (const char*)other + (size_t)g * cg * es_x : (const char*)w + (size_t)g * og * es_w;
    char* c = (char*)out + (size_t)g * (pass == 0 ? og * es_y : (pass == 1 ? cg * es_x : og * es_w));
    gb_epilogue slice = {};
    if (ep) {
      slice = *ep;
      if (ep->bias) slice.bias = ep->bias + (size_t)g * og;
      if (ep->residual) slice.residual = (const char*)ep->residual + (size_t)g * og * es_y;
    }
    const PlanKey key = make_key(0x100u + (uint32_t)pass, &one, sizeof(one), a, b, c, ep ? &slice : nullptr, workspace, workspace_bytes);
    const Plan* cached = cache_find(h, key);
    Plan plan;
    if (!cached) {
      int rc = plan_conv(h, pass, &one, a, b, c, ep ? &slice : nullptr, plan, nullptr, nullptr, nullptr, o_total, o_total);
      if (rc == GB_OK) rc = prepare_plan(h, plan, workspace, workspace_bytes);
      if (rc != GB_OK) return rc;
      cache_store(h, key, plan);
      cached = &plan;
    }
    const int rc = launch_plan(h, stream, *cached);
    if (rc != GB_OK) return rc;
    launches += h->last_plan.kernel_launches;
    items += h->last_plan.work_items;
  }
  h->last_plan.kernel_launches = launches + extra;
  h->last_plan.work_items = items;
  return GB_OK;
}

}  // namespace

// =====================================================================================================
extern "C" {

int gb_abi_version(void) { return GB_ABI_VERSION; }

const char* gb_error_string(int status) {
  switch (status) {
    case GB_OK: return "success";
    case GB_ERR_INVALID: return "invalid argument";
    case GB_ERR_CUDA: return "a CUDA call failed";
    case GB_ERR_WORKSPACE: return "workspace missing or too small";
    case GB_ERR_UNSUPPORTED: return "shape or dtype combination not supported";
    case GB_ERR_TIMEOUT: return "a bounded device-side wait gave up";
    case GB_ERR_NCCL: return "NCCL unavailable or a collective failed";
    case GB_ERR_NO_DEVICE: return "no sm_100 CUDA device";
    default: return "unknown status";
  }
}

int gb_create(int device_ordinal, gb_handle** out) {
  if (!out) return GB_ERR_INVALID;
  *out = nullptr;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || device_ordinal < 0 || device_ordinal >= count) return GB_ERR_NO_DEVICE;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device_ordinal) != cudaSuccess) return GB_ERR_NO_DEVICE;
  if (prop.major != 10) return GB_ERR_NO_DEVICE;   // the kernels are sm_100a only; there is no fallback
  if (cudaSetDevice(device_ordinal) != cudaSuccess) return GB_ERR_CUDA;
  gb_handle* h = new gb_handle();
  h->device = device_ordinal;
  h->sm_count = prop.multiProcessorCount;
  cudaError_t e = cudaMalloc(&h->status, sizeof(uint32_t));
  if (e == cudaSuccess) e = cudaMemset(h->status, 0, sizeof(uint32_t));
  h->test_drops_left = knobs().test_drop_calls;
  if (e == cudaSuccess) e = gb::gemm_sm100_configure();
  if (e != cudaSuccess || encode_tiled_fn() == nullptr) {
    if (h->status) cudaFree(h->status);
    delete h;
    return GB_ERR_CUDA;
  }
  *out = h;
  return GB_OK;
}

void gb_destroy(gb_handle* h) {
  if (!h) return;
  cudaSetDevice(h->device);
  if (h->status) cudaFree(h->status);
  delete h;
}

int gb_last_cuda_error(const gb_handle* h) { return h ? h->last_cuda : 0; }
int gb_sm_count(const gb_handle* h) { return h ? h->sm_count : 0; }

int gb_last_status(gb_handle* h, void* stream, uint32_t* device_status) {
  if (!h) return GB_ERR_INVALID;
  uint32_t word = 0;
  cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaMemcpy(&word, h->status, sizeof(word), cudaMemcpyDeviceToHost);
  if (e == cudaSuccess && word != 0) e = cudaMemset(h->status, 0, sizeof(word));
  if (e != cudaSuccess) return cuda_fail(h, e);
  if (device_status) *device_status = word;
  return word == 0 ? GB_OK : GB_ERR_TIMEOUT;
}

uint64_t gb_plan_cache_hits(const gb_handle* h) { return h ? h->cache_hits : 0; }

int gb_last_plan(const gb_handle* h, gb_plan_info* out) {
  if (!h || !out) return GB_ERR_INVALID;
  *out = h->last_plan;
  return GB_OK;
}

int gb_gemm_workspace(const gb_handle* h, const gb_gemm_desc* desc, size_t* bytes) {
  if (!h || !bytes) return GB_ERR_INVALID;
  int rc = validate_gemm(desc);
  if (rc != GB_OK) return rc;
  gb_handle* hm = const_cast<gb_handle*>(h);   // the cache is bookkeeping, not state a caller can observe
  const PlanKey key = make_key(0x10, desc, sizeof(*desc), nullptr, nullptr, nullptr, nullptr, nullptr, 0);
  if (const Plan* cached = cache_find(hm, key)) {
    *bytes = cached->workspace;
    return GB_OK;
  }
  Plan plan;
  rc = plan_gemm(h, desc, nullptr, nullptr, nullptr, nullptr, plan);
  if (rc != GB_OK) return rc;
  // room for the ordered batch-norm statistics of a call whose epilogue asks for them (the query does not see the epilogue)
  plan.workspace = std::max(plan.workspace, (size_t)h->sm_count * kStatsPartialBytesPerCta);
  cache_store(hm, key, plan);
  *bytes = plan.workspace;
  return GB_OK;
}

int gb_gemm(gb_handle* h, void* stream, const gb_gemm_desc* desc, const void* a, const void* b, void* c,
            const gb_epilogue* epilogue, void* workspace, size_t workspace_bytes) {
  if (!h) return GB_ERR_INVALID;
  int rc = validate_gemm(desc);
  if (rc != GB_OK) return rc;
  if (desc->m != 0 && desc->n != 0 && (!c || (desc->k != 0 && (!a || !b)))) return GB_ERR_INVALID;
  const PlanKey key = make_key(0, desc, sizeof(*desc), a, b, c, epilogue, workspace, workspace_bytes);
  if (const Plan* cached = cache_find(h, key)) return launch_plan(h, (cudaStream_t)stream, *cached);
  Plan plan;
  rc = plan_gemm(h, desc, a, b, c, epilogue, plan);
  if (rc == GB_OK) rc = prepare_plan(h, plan, workspace, workspace_bytes);
  if (rc != GB_OK) return rc;
  cache_store(h, key, plan);
  return launch_plan(h, (cudaStream_t)stream, plan);
}

int gb_conv_workspace(const gb_handle* h, int pass, const gb_conv_desc* desc, size_t* bytes) {
  if (!h || !bytes || pass < 0 || pass > 2) return GB_ERR_INVALID;
  int rc = validate_conv(desc);
  if (rc != GB_OK) return rc;
  Plan plan;
  gb_conv_desc shadow;
  size_t head = 0;
  if (pass != 2 && wants_filter_shadow(desc)) {
    shadow = *desc;
    shadow.dtype_w = GB_BF16;
    desc = &shadow;
    head = filter_shadow_bytes(desc);
  }
  gb_conv_desc one;
  uint32_t y_step = 0;
  if (desc->groups > 1) {   // every group runs the same plan: one group's need
    one = *desc;
    y_step = desc->geo.c_out;
    one.geo.c_step = desc->geo.c_step ? desc->geo.c_step : desc->geo.c;
    one.geo.c = desc->geo.c / desc->groups;
    one.geo.c_out = desc->geo.c_out / desc->groups;
    one.groups = 1;
    desc = &one;
  }
  gb_handle* hm = const_cast<gb_handle*>(h);
  const PlanKey key = make_key(0x11 + (uint32_t)pass, desc, sizeof(*desc), nullptr, nullptr, nullptr, nullptr, nullptr, 0);
  if (const Plan* cached = cache_find(hm, key)) {
    *bytes = head + cached->workspace;
    return GB_OK;
  }
  rc = plan_conv(h, pass, desc, nullptr, nullptr, nullptr, nullptr, plan, nullptr, nullptr, nullptr, y_step, y_step);
  if (rc != GB_OK) return rc;
  if (pass != 2) plan.workspace = std::max(plan.workspace, (size_t)h->sm_count * kStatsPartialBytesPerCta);   // ordered statistics, if asked for
  if (pass != 1) plan.workspace += ((size_t)desc->geo.c * 4 + 255) & ~(size_t)255;                              // the expanded norm of the *_affine entry points
  cache_store(hm, key, plan);
  *bytes = head + plan.workspace;
  return GB_OK;
}

int gb_conv_fprop(gb_handle* h, void* stream, const gb_conv_desc* desc, const void* x, const void* w, void* y,
                  const gb_epilogue* epilogue, void* workspace, size_t workspace_bytes) {
  if (!h || !x || !w || !y) return GB_ERR_INVALID;
  int rc = validate_conv(desc);
  if (rc != GB_OK) return rc;
  if (desc->groups > 1) return run_grouped(h, (cudaStream_t)stream, 0, desc, x, w, y, epilogue, workspace, workspace_bytes);
  gb_conv_desc shadow;
  rc = make_filter_shadow(h, (cudaStream_t)stream, desc, shadow, w, workspace, workspace_bytes);
  if (rc != GB_OK) return rc;
  const PlanKey key = make_key(1, desc, sizeof(*desc), x, w, y, epilogue, workspace, workspace_bytes);
  const Plan* cached = cache_find(h, key);
  Plan plan;
  if (!cached) {
    rc = plan_conv(h, 0, desc, x, w, y, epilogue, plan);
    if (rc == GB_OK) rc = prepare_plan(h, plan, workspace, workspace_bytes);
    if (rc != GB_OK) return rc;
    cache_store(h, key, plan);
    cached = &plan;
  }
  rc = launch_plan(h, (cudaStream_t)stream, *cached);
  if (desc == &shadow) h->last_plan.kernel_launches += 1;   // the cast of the filters
  return rc;
}

int gb_conv_dgrad(gb_handle* h, void* stream, const gb_conv_desc* desc, const void* dy, const void* w, void* dx,
                  void* workspace, size_t workspace_bytes) {
  if (!h || !dy || !w || !dx) return GB_ERR_INVALID;
  int rc = validate_conv(desc);
  if (rc != GB_OK) return rc;
  if (desc->w_layout != 0) return GB_ERR_UNSUPPORTED;   // the prepared filter copy is a forward-only format
  if (desc->groups > 1) return run_grouped(h, (cudaStream_t)stream, 1, desc, dy, w, dx, nullptr, workspace, workspace_bytes);
  gb_conv_desc shadow;
  rc = make_filter_shadow(h, (cudaStream_t)stream, desc, shadow, w, workspace, workspace_bytes);
  if (rc != GB_OK) return rc;
  const uint32_t extra = desc == &shadow ? 1u : 0u;   // the cast of the filters
  if (desc->geo.stride > 1) {
    rc = run_dgrad_classes(h, (cudaStream_t)stream, desc, dy, w, dx);
    if (rc != GB_ERR_UNSUPPORTED) {
      if (rc == GB_OK) h->last_plan.kernel_launches += extra;
      return rc;
    }
  }
  const PlanKey key = make_key(2, desc, sizeof(*desc), dy, w, dx, nullptr, workspace, workspace_bytes);
  const Plan* cached = cache_find(h, key);
  Plan plan;
  if (!cached) {
    rc = plan_conv(h, 1, desc, dy, w, dx, nullptr, plan);
    if (rc == GB_OK) rc = prepare_plan(h, plan, workspace, workspace_bytes);
    if (rc != GB_OK) return rc;
    cache_store(h, key, plan);
    cached = &plan;
  }
  rc = launch_plan(h, (cudaStream_t)stream, *cached);
  h->last_plan.kernel_launches += extra;
  return rc;
}

namespace {
// Carves the bf16 scale / shift vectors of the expanded norm out of the head of the workspace; returns what is left of it.
int carve_affine(const gb_affine_input* affine, uint32_t c, void*& workspace, size_t& workspace_bytes, uint16_t*& scale, uint16_t*& shift) {
  if (!affine || !affine->mean || !affine->inv_std || !affine->gamma || !affine->beta) return GB_ERR_INVALID;
  const size_t need = ((size_t)c * 4 + 255) & ~(size_t)255;
  if (workspace == nullptr || workspace_bytes < need || !aligned16(workspace)) return GB_ERR_WORKSPACE;
  scale = (uint16_t*)workspace;
  shift = scale + ((c + 7) & ~7u);
  workspace = (char*)workspace + need;
  workspace_bytes -= need;
  return GB_OK;
}

// Plans, prepares and launches a pass over a virtual normalised input.  Where the transform warps take the operand they
// expand the norm themselves (a table in shared memory); otherwise the expansion kernel fills the workspace vectors first.
int run_affine(gb_handle* h, cudaStream_t stream, int pass, const gb_conv_desc* desc, const void* act, const void* other, void* out,
               const gb_epilogue* epilogue, const gb_affine_input* affine, uint16_t* scale, uint16_t* shift, void* workspace, size_t workspace_bytes) {
  Plan plan;
  int rc = plan_conv(h, pass, desc, act, other, out, epilogue, plan, nullptr, scale, shift);
  if (rc != GB_OK) return rc;
  const bool own_table = plan.p.xform != 0;
  if (own_table) {
    plan.p.aff_mean = affine->mean; plan.p.aff_inv_std = affine->inv_std; plan.p.aff_gamma = affine->gamma; plan.p.aff_beta = affine->beta;
  }
  rc = prepare_plan(h, plan, workspace, workspace_bytes);
  if (rc != GB_OK) return rc;
  if (!own_table) {
    const cudaError_t e = gb::launch_affine_expand(affine->mean, affine->inv_std, affine->gamma, affine->beta, scale, shift, desc->geo.c, stream);
    if (e != cudaSuccess) return cuda_fail(h, e);
  }
  rc = launch_plan(h, stream, plan);
  h->last_plan.kernel_launches += own_table ? 0 : 1;
  return rc;
}
}  // namespace

int gb_conv_fprop_affine(gb_handle* h, void* stream, const gb_conv_desc* desc, const void* x, const void* w, void* y,
                         const gb_epilogue* epilogue, const gb_affine_input* affine, void* workspace, size_t workspace_bytes) {
  if (!h || !x || !w || !y) return GB_ERR_INVALID;
  int rc = validate_conv(desc);
  if (rc != GB_OK) return rc;
  if (desc->groups > 1) return GB_ERR_UNSUPPORTED;
  uint16_t *scale = nullptr, *shift = nullptr;
  rc = carve_affine(affine, desc->geo.c, workspace, workspace_bytes, scale, shift);
  if (rc != GB_OK) return rc;
  gb_conv_desc shadow;
  rc = make_filter_shadow(h, (cudaStream_t)stream, desc, shadow, w, workspace, workspace_bytes);
  if (rc != GB_OK) return rc;
  const bool cast = desc == &shadow;
  rc = run_affine(h, (cudaStream_t)stream, 0, desc, x, w, y, epilogue, affine, scale, shift, workspace, workspace_bytes);
  if (rc == GB_OK && cast) h->last_plan.kernel_launches += 1;
  return rc;
}

int gb_conv_wgrad_affine(gb_handle* h, void* stream, const gb_conv_desc* desc, const void* dy, const void* x, void* dw,
                         const gb_affine_input* affine, void* workspace, size_t workspace_bytes) {
  if (!h || !dy || !x || !dw) return GB_ERR_INVALID;
  int rc = validate_conv(desc);
  if (rc != GB_OK) return rc;
  if (desc->dtype_w != GB_F32 || desc->w_layout != 0 || desc->groups > 1) return GB_ERR_UNSUPPORTED;
  uint16_t *scale = nullptr, *shift = nullptr;
  rc = carve_affine(affine, desc->geo.c, workspace, workspace_bytes, scale, shift);
  if (rc != GB_OK) return rc;
  return run_affine(h, (cudaStream_t)stream, 2, desc, dy, x, dw, nullptr, affine, scale, shift, workspace, workspace_bytes);
}

int gb_conv_dgrad_stats(gb_handle* h, void* stream, const gb_conv_desc* desc, const void* dy, const void* w, void* dx,
                        const gb_dx_stats* stats, void* workspace, size_t workspace_bytes) {
  if (!stats) return gb_conv_dgrad(h, stream, desc, dy, w, dx, workspace, workspace_bytes);
  if (!h || !dy || !w || !dx) return GB_ERR_INVALID;
  int rc = validate_conv(desc);
  if (rc != GB_OK) return rc;
  if (desc->w_layout != 0 || desc->groups > 1) return GB_ERR_UNSUPPORTED;
  gb_conv_desc shadow;
  rc = make_filter_shadow(h, (cudaStream_t)stream, desc, shadow, w, workspace, workspace_bytes);
  if (rc != GB_OK) return rc;
  Plan plan;
  rc = plan_conv(h, 1, desc, dy, w, dx, nullptr, plan, stats);
  if (rc == GB_OK) rc = prepare_plan(h, plan, workspace, workspace_bytes);
  if (rc != GB_OK) return rc;
  rc = launch_plan(h, (cudaStream_t)stream, plan);
  if (desc == &shadow) h->last_plan.kernel_launches += 1;
  return rc;
}

int gb_conv_wgrad(gb_handle* h, void* stream, const gb_conv_desc* desc, const void* dy, const void* x, void* dw,
                  void* workspace, size_t workspace_bytes) {
  if (!h || !dy || !x || !dw) return GB_ERR_INVALID;
  int rc = validate_conv(desc);
  if (rc != GB_OK) return rc;
  if (desc->dtype_w != GB_F32 || desc->w_layout != 0) return GB_ERR_UNSUPPORTED;   // weight gradients accumulate in f32 (gpu.zig:983)
  if (desc->groups > 1) return run_grouped(h, (cudaStream_t)stream, 2, desc, dy, x, dw, nullptr, workspace, workspace_bytes);
  const PlanKey key = make_key(3, desc, sizeof(*desc), dy, x, dw, nullptr, workspace, workspace_bytes);
  if (const Plan* cached = cache_find(h, key)) return launch_plan(h, (cudaStream_t)stream, *cached);
  Plan plan;
  rc = plan_conv(h, 2, desc, dy, x, dw, nullptr, plan);
  if (rc == GB_OK) rc = prepare_plan(h, plan, workspace, workspace_bytes);
  if (rc != GB_OK) return rc;
  cache_store(h, key, plan);
  return launch_plan(h, (cudaStream_t)stream, plan);
}

}  // extern "C"

// =====================================================================================================
// gb_gemm_static_scratch: the product of gb_gemm for callers that must not allocate device memory.
//
// Some hosts of this library run where cudaMalloc is off limits: a plugin whose memory is owned by an
// arena that hands out nothing after start-up, or a process with a fixed device-memory budget.  gb_gemm needs two things such a caller cannot provide: a
// handle (gb_create allocates a status word) and, when K is split, a workspace for the partial sums.  This
// entry point needs neither.  Its split-K partials live in the array below, which is part of the library
// image: every GPU that loads the library carries these 4 MiB until the process exits.
//
// The array's name is only a stand-in on the host; the kernels need its device address, which is looked up
// once per device with cudaGetSymbolAddress while that device is current.  That look-up happens on the
// first call made with a given device current, so make that first call outside any stream capture.
// All calls share the one array and it keeps whatever the previous call left: every element a call reads
// is written by the same call first (each K part stores its whole partial tile), so nothing has to be
// cleared, but two calls that overlap on the GPU -- different streams, or different host threads -- race on
// it.  Serialise them.  A bounded device-side wait that gives up is reported into a status word that also lives in
// the library image; gb_static_last_status reads and clears it.
namespace {

__device__ __align__(256) unsigned char g_static_scratch[GB_STATIC_SCRATCH_BYTES];
// The word a kernel launched by this entry point reports a bounded wait that gave up into (0 = none); read and
// cleared by gb_static_last_status.  Like the array it belongs to the library image, one copy per GPU.
__device__ uint32_t g_static_status;

constexpr int kMaxStaticDevices = 64;
std::mutex g_static_mutex;
void* g_static_scratch_ptr[kMaxStaticDevices] = {};
uint32_t* g_static_status_ptr[kMaxStaticDevices] = {};
int g_static_sm_count[kMaxStaticDevices] = {};

// Resolves the device addresses of the scratch array and the status word for the current device (once), without allocating.
int static_setup(int device, void** scratch, uint32_t** status, int* sm_count) {
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (device < 0 || device >= kMaxStaticDevices) return GB_ERR_NO_DEVICE;
  if (g_static_scratch_ptr[device] == nullptr) {
    int major = 0, sms = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess || major != 10) return GB_ERR_NO_DEVICE;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return GB_ERR_CUDA;
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || ptr == nullptr) return GB_ERR_CUDA;
    void* word = nullptr;
    if (cudaGetSymbolAddress(&word, g_static_status) != cudaSuccess || word == nullptr) return GB_ERR_CUDA;
    if (gb::gemm_sm100_configure() != cudaSuccess || encode_tiled_fn() == nullptr) return GB_ERR_CUDA;
    g_static_sm_count[device] = sms;
    g_static_status_ptr[device] = (uint32_t*)word;
    g_static_scratch_ptr[device] = ptr;
  }
  *scratch = g_static_scratch_ptr[device];
  *status = g_static_status_ptr[device];
  *sm_count = g_static_sm_count[device];
  return GB_OK;
}

}  // namespace

extern "C" int gb_gemm_static_scratch(void* stream, const gb_gemm_desc* desc, const void* a, const void* b, void* c,
                                      const gb_epilogue* epilogue) {
  int rc = validate_gemm(desc);
  if (rc != GB_OK) return rc;
  if (desc->m != 0 && desc->n != 0 && (!c || (desc->k != 0 && (!a || !b)))) return GB_ERR_INVALID;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return GB_ERR_NO_DEVICE;
  void* scratch = nullptr;
  gb_handle local;            // lives on the host stack (so nothing is cached); its status word is the one inside the library image
  local.device = device;
  rc = static_setup(device, &scratch, &local.status, &local.sm_count);
  if (rc != GB_OK) return rc;
  Plan plan;
  rc = plan_gemm(&local, desc, a, b, c, epilogue, plan);
  if (rc != GB_OK) return rc;
  // A product whose partial sums do not fit the fixed array is refused, not silently run another way.
  if (plan.workspace > (size_t)GB_STATIC_SCRATCH_BYTES) return GB_ERR_WORKSPACE;
  return run_plan(&local, (cudaStream_t)stream, plan, scratch, GB_STATIC_SCRATCH_BYTES);
}

extern "C" int gb_static_last_status(void* stream, uint32_t* device_status) {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return GB_ERR_NO_DEVICE;
  void* scratch = nullptr;
  uint32_t* status = nullptr;
  int sms = 0;
  int rc = static_setup(device, &scratch, &status, &sms);
  if (rc != GB_OK) return rc;
  uint32_t word = 0;
  cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaMemcpy(&word, status, sizeof(word), cudaMemcpyDeviceToHost);
  if (e == cudaSuccess && word != 0) e = cudaMemset(status, 0, sizeof(word));
  if (e != cudaSuccess) return GB_ERR_CUDA;
  if (device_status) *device_status = word;
  return word == 0 ? GB_OK : GB_ERR_TIMEOUT;
}
