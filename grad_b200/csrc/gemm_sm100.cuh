// Parameter block shared by the host dispatcher and the tcgen05 contraction kernel.
#pragma once

#include <cuda.h>
#include <cstdlib>
#include <utility>
#include <cuda_runtime.h>
#include <stdint.h>

namespace gb {

// How one operand's tile reaches shared memory.
enum OperandKind : uint32_t {
  kDenseK = 0,      // TMA, K contiguous in memory: lines = MN index, 128 B of K per line
  kDenseMN = 1,     // TMA, MN contiguous in memory: blocks of `epl` MN values, one line per K index
  kPatchK = 2,      // TMA over NHWC activations, lines = output positions, 128 B of channels per line (conv A, K-major)
  kPatchMN = 3,     // same boxes read as MN-major A: lines = positions (K), 128 B of (tap, channel) per line (wgrad)
  kWeightK = 4,     // TMA over weights viewed (c_out, c_in, taps): lines = c_in (N), 128 B of c_out (K) (dgrad B)
  kGather = 5,      // filled by the gather warps with plain loads (any stride, dtype or geometry)
};

// What the gather warps read when an operand is kGather.
enum GatherSource : uint32_t {
  kSrcDense = 0,    // element(line_major, inner) = base[line_major * ld + inner]
  kSrcPatch = 1,    // lines = positions, inner = (tap, channel): the implicit im2col matrix of x
  kSrcPatchT = 2,   // zero-insertion gather of dy for the input gradient of a strided convolution
  kSrcWeightT = 3,  // lines = c_in, inner = (flipped tap, c_out): w read transposed for the input gradient
};

struct ConvGeo {
  uint32_t n, h, w, c, k, stride, pad, dilation, out_h, out_w, c_out, c_step;
  // Channel pitch of y / dy and column pitch of w / dw in memory: c_out for a dense layer; one group of a grouped layer
  // is a layer of its own over channel slices of x, w and y, whose pitches stay those of the whole tensors.
  uint32_t y_step, w_step;
};

struct GatherDesc {
  const void* base;
  uint64_t batch_stride;   // elements
  uint32_t source;         // GatherSource
  uint32_t src_is_bf16;    // storage type in global memory
  uint32_t ld;             // dense: row pitch in elements
  uint32_t lines_total;    // bound on the line-major index (rows that exist)
  uint32_t inner_total;    // bound on the inner index
  uint32_t mn_major;       // 1: lines are K indices and inner is MN; 0: lines are MN and inner is K
};

// Division by a run-time constant without the ~100-cycle integer divide: an under-estimate from the high
// product with floor((2^32 - 1) / d), then at most two corrections (device side: `fast_div`).
struct FastDiv {
  uint32_t d, m;
};
inline FastDiv make_fastdiv_host(uint32_t d) { return FastDiv{d ? d : 1u, 0xFFFFFFFFu / (d ? d : 1u)}; }

// How a patch operand (kPatchK) and the filter operand of an input gradient (kWeightK) walk along K: channel
// blocks innermost, then `n1` taps along x, then the taps along y.  A forward pass, a stride-1 input gradient
// and one parity class of a strided input gradient differ only in these numbers.
struct TapWalk {
  uint32_t cblocks, n1, n2;    // channel blocks per tap; taps along x; taps along y
  uint32_t grid_h, grid_w;     // a tile's rows enumerate (image, i, j) over this grid
  FastDiv div_image, div_w;    // dividers by grid_h * grid_w and by grid_w
  uint32_t row_scale;          // patch row of grid row i at the first tap: i * row_scale + z0
  int32_t y0, z0;              // patch column / row of grid position (0, 0) at the first tap
  int32_t y_step, z_step;      // patch column step per tap along x, patch row step per tap along y
  int32_t tap0, tap_x, tap_y;  // filter tap index: first tap, step per tap along x, step per tap along y
};

// Where row m of the product lands when it is not row m of C: one parity class of a strided input gradient
// writes pixel (image, i * scale + off_y, j * scale + off_x) of an NHWC tensor for row (image, i, j).
struct RowMap {
  uint32_t enabled;
  FastDiv per_image, grid_w;
  uint32_t h, w, scale, off_y, off_x;
};

// One parity class of a fused strided input gradient (see `GemmParams::n_classes`).
struct ClassSlot {
  TapWalk walk;
  RowMap rowmap;
  uint32_t m, k_blocks;   // rows and K blocks of this class's product
};
constexpr uint32_t kMaxClasses = 4;

struct GemmParams {
  // problem
  uint32_t m, n, k, batch;
  uint32_t tiles_m, tiles_n, splits, k_blocks_per_split, k_blocks_total;
  uint32_t bn;              // tile columns (multiple of 32, <= 256)
  uint32_t stages;
  uint32_t k_mul;           // > 1: both operands are MN-major TMA tiles and a stage holds k_mul K blocks (boxes of k_mul times as many lines)
  uint32_t tf32;            // 1: kind::tf32 on f32 tiles (32 elements per line), 0: kind::f16 on bf16 tiles (64 per line)
  uint32_t a_kind, b_kind;  // OperandKind
  uint32_t a_mn_major, b_mn_major;
  uint32_t group_m;         // tile rasterisation band height
  FastDiv div_splits, div_per_batch, div_band, div_group;   // dividers of the work decode: splits, tiles_m * tiles_n, group_m * tiles_n, group_m
  uint32_t cta_pair;        // 1: two CTAs share a 256 x bn tile (tiles_m counts 256-row tiles)
  // TMA patch boxes (conv): positions per box and its decomposition
  uint32_t box_w, box_h, box_n;
  ConvGeo geo;
  uint32_t dgrad;           // 1: patches are taken from dy with flipped taps (input gradient)
  // s > 1: the only parity class of a strided input gradient that has taps (a 1x1 layer of stride s); its epilogue also
  // writes the zeros of the s*s - 1 pixels beside each of its pixels, which saves clearing dx in front of the launch
  uint32_t zero_fill;
  uint32_t patch_view;      // 1: the activation map is already a strided view of x (1x1 strided layer): MN-major patch boxes step rows by 1
  TapWalk walk;             // K walk of patch / filter-tap boxes
  // Column-patch stages (col_taps > 0): one stage holds, for one (tap column, channel block), the activation
  // rows that ALL col_taps taps of that column read -- box_h + (col_taps - 1) * |row step| image rows in one
  // box -- and one B tile per tap; tap t's A operand starts col_a_first16 + t * col_a_step16 (bytes >> 4)
  // into the A part.  K blocks then count (tap column, channel block) pairs.
  uint32_t col_taps;
  uint32_t a_stage_bytes;   // A part of a stage (multiple of 1024); 0 means the plain 16 KB tile
  uint32_t a_box_bytes;     // bytes the A box really delivers
  int32_t col_a_first16, col_a_step16;
  RowMap rowmap;            // output row placement (disabled: row m of C)
  // > 0: the batch index selects one of `n_classes` products that share operands, tile shape and C but have their
  // own tap walk, row map, row count and K length (the parity classes of a strided input gradient in one launch)
  uint32_t n_classes;
  ClassSlot cls[kMaxClasses];
  // gather sources
  GatherDesc ga, gbsrc;
  // non-null: the patch operand stands for relu(scale[ci] * x + shift[ci]) of the stored bf16 map (a batch norm and ReLU
  // that were never written out); bf16[c] each, applied by the gather warps to in-bounds taps only (padding stays zero)
  const uint16_t* affine_scale;
  const uint16_t* affine_shift;
  // 1: the A operand stands for relu(scale * x + shift) and arrives by TMA with out-of-bounds elements filled with NaN;
  // the two extra warps rewrite each landed A tile in place (NaN -> 0: padding stays zero) and only then hand the stage to
  // the MMA issuer.  0 with affine_scale set: the gather warps apply the transform while they build the tile.
  uint32_t xform;
  // with xform (always set then): the four per-channel vectors of the norm (f32[c], c <= kMaxXformTableChannels).  The
  // transform warps expand them into a table in shared memory at kernel start (s = gamma * inv_std, t = beta - mean * s,
  // each rounded to bf16: `affineExpand`, src/gpu/device.zig:1774-1783), which saves the expansion launch;
  // affine_scale / affine_shift are not read then.
  const float* aff_mean;
  const float* aff_inv_std;
  const float* aff_gamma;
  const float* aff_beta;
  // output
  void* c;
  const float* bias;
  const void* residual;
  float* partial;           // split-K partials: [split][batch][m][n] f32, dense
  uint64_t stride_c;        // batch stride of C in elements
  // Two batch levels (batch_inner != 0): work item b is product (b / batch_inner, b % batch_inner); operand maps carry the
  // outer level as their fourth dimension, C as its fourth dimension or through stride_c_outer.
  uint64_t stride_c_outer;
  uint32_t batch_inner;
  FastDiv div_batch_inner;
  uint32_t ldc;
  uint32_t c_is_bf16, transpose_out, accumulate, relu, vec_store;
  uint32_t epi_groups;      // epilogue warps = 4 * epi_groups; group g drains column chunks g, g + groups, ...
  uint32_t round_tf32;      // round the stored f32 result to TF32 (nearest, ties away)
  uint32_t tma_store;       // full 32-column chunks leave through shared memory and a TMA store (map of C passed to the kernel)
  // batch-norm statistics of the stored result, summed in the epilogue (stats != 0): see `chunk_stats`
  uint32_t stats;           // 1: forward sums of (v - shift), (v - shift)^2; 2: backward sums of the masked gradient g and g * x_hat
  const float* stat_shift;  // f32[n]: the values are centred by it before they are summed (mode 2: the batch mean)
  const void* stat_x;       // mode 2: the raw bf16 map the norm ran on, laid out like the result
  const float *stat_inv_std, *stat_gamma, *stat_beta;   // mode 2: f32[n] each
  float* stat_sums;         // f32[2n]: += sum(v - shift), += sum((v - shift)^2)
  float* stat_partial;      // ordered runs: [cta][8 warps][4 chunks][32 lanes][2], combined by `stats_combine_kernel`; else null
  uint32_t* status;
  uint32_t spin_limit;      // failed polls after which a bounded wait gives up (0 = the default, about a second)
  uint32_t test_drop_kblock;   // fault injection on the host's request: the producer leaves out this K block's copies (+1; 0 = off)
};

// Threads of the gather warps (single-CTA kernel, plans with a gathered operand).  Two warps: with four the CTA had 14
// warps, four of them on one scheduler, which caps every thread at 128 registers and spilled the epilogue of EVERY
// plan of that kernel; 12 warps leave 168.
constexpr uint32_t kGatherThreads = 64;
// Shared memory the epilogue warps own when p.tma_store is set: per warp a 2 KB staging block (32 rows x 64
// bytes, 64-byte swizzle) and 1 KB of bias values (eight 32-column chunks).
constexpr uint32_t kStoreStageBytesPerWarp = 2048;
constexpr uint32_t kStoreBiasBytesPerWarp = 1024;
constexpr uint32_t kStoreSmemBytes = 8 * (kStoreStageBytesPerWarp + kStoreBiasBytesPerWarp);
// statistics plans: per epilogue warp the per-column values of its four column chunks (4 x 512 B) and its running sums (1 KB), behind the block above
constexpr uint32_t kStatBytesPerWarp = 4 * 512 + 1024;
constexpr uint32_t kMaxXformTableChannels = 2048;   // 8 KB of shared memory for the scale and shift tables
// Launch with programmatic stream serialization (the kernel must execute griddepcontrol.wait before its first
// global access).  GB_NO_OVERLAPPED_LAUNCH=1 falls back to plain stream order.
template <class... KernelArgs, class... Args>
inline cudaError_t launch_overlapped(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  static const bool plain = getenv("GB_NO_OVERLAPPED_LAUNCH") != nullptr;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = plain ? 0 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

size_t gemm_smem_bytes(const GemmParams& p);
cudaError_t launch_gemm_sm100(const GemmParams& p, const CUtensorMap& tmap_a, const CUtensorMap& tmap_b, const CUtensorMap& tmap_c, int sm_count,
                              cudaStream_t stream);
cudaError_t launch_splitk_reduce(const GemmParams& p, cudaStream_t stream);
uint32_t gemm_grid_ctas(const GemmParams& p, int sm_count);
cudaError_t launch_stats_combine(const GemmParams& p, uint32_t ctas, cudaStream_t stream);
cudaError_t gemm_sm100_configure();
uint32_t f32_grid_blocks(const GemmParams& p, uint32_t tm, uint32_t tn);

}  // namespace gb
