// Strict-f32 contraction on the CUDA cores: the GB_MATH_F32 path.  One kernel covers the dense matmul
// family in every layout and the three convolution passes, because both operands are read through the
// same (line, inner) element accessors the tensor-core kernel's gather warps use.  Every product is an
// f32 FMA into an f32 accumulator, K ascending within a split -- the arithmetic of grad's `Gemm`
// (src/gpu/device.zig:122-201) and `f32Compute` (:1665-1684).
#include "gemm_sm100.cuh"
#include "sm100_ptx.cuh"

namespace gb {

namespace {

constexpr uint32_t kTM = 64, kTN = 64, kTK = 16;

__device__ __forceinline__ int64_t f32_gather_index(const GatherDesc& d, const ConvGeo& g, uint32_t line, uint32_t inner) {
  if (line >= d.lines_total || inner >= d.inner_total) return -1;
  switch (d.source) {
    case kSrcDense:
      return (int64_t)line * d.ld + inner;
    case kSrcPatch: {
      const uint32_t tap = inner / g.c, ci = inner - tap * g.c;
      const uint32_t ky = tap / g.k, kx = tap - ky * g.k;
      const uint32_t per_image = g.out_h * g.out_w;
      const uint32_t n = line / per_image, rem = line - n * per_image;
      const uint32_t oy = rem / g.out_w, ox = rem - oy * g.out_w;
      const uint32_t py = oy * g.stride + ky * g.dilation, px = ox * g.stride + kx * g.dilation;
      if (py < g.pad || px < g.pad || py - g.pad >= g.h || px - g.pad >= g.w) return -1;
      return ((int64_t)(n * g.h + py - g.pad) * g.w + px - g.pad) * g.c_step + ci;
    }
    case kSrcPatchT: {
      const uint32_t tap = inner / g.c_out, co = inner - tap * g.c_out;
      const uint32_t ky = tap / g.k, kx = tap - ky * g.k;
      const uint32_t per_image = g.h * g.w;
      const uint32_t n = line / per_image, rem = line - n * per_image;
      const uint32_t y = rem / g.w, x = rem - y * g.w;
      const int32_t ty = (int32_t)(y + g.pad) - (int32_t)(ky * g.dilation);
      const int32_t tx = (int32_t)(x + g.pad) - (int32_t)(kx * g.dilation);
      if (ty < 0 || tx < 0) return -1;
      const uint32_t oy = (uint32_t)ty / g.stride, ox = (uint32_t)tx / g.stride;
      if (oy * g.stride != (uint32_t)ty || ox * g.stride != (uint32_t)tx || oy >= g.out_h || ox >= g.out_w) return -1;
      return ((int64_t)(n * g.out_h + oy) * g.out_w + ox) * g.y_step + co;
    }
    default: {
      const uint32_t tap = inner / g.c_out, co = inner - tap * g.c_out;
      return ((int64_t)tap * g.c + line) * g.w_step + co;
    }
  }
}

__device__ __forceinline__ float f32_operand(const GatherDesc& d, const ConvGeo& g, uint64_t batch_off, uint32_t mn, uint32_t kk) {
  const int64_t idx = d.mn_major ? f32_gather_index(d, g, kk, mn) : f32_gather_index(d, g, mn, kk);
  if (idx < 0) return 0.0f;
  return d.src_is_bf16 ? bf16_to_f32(((const uint16_t*)d.base)[batch_off + idx]) : ((const float*)d.base)[batch_off + idx];
}

// Which tile a block owns.  The grid is one-dimensional, column tiles innermost, then row tiles, then (batch, K
// part): grid.y and grid.z stop at 65535, which a convolution over 4096 images of 32 x 32 outputs (65536 row
// tiles) already exceeds; grid.x does not.
struct TileIndex {
  uint32_t m0, n0, split, batch;
};
template <uint32_t TM, uint32_t TN>
__device__ __forceinline__ TileIndex f32_tile_index(const GemmParams& p) {
  const uint32_t tiles_n = (p.n + TN - 1) / TN, tiles_m = (p.m + TM - 1) / TM;
  uint32_t w = blockIdx.x;
  const uint32_t tn = w % tiles_n;
  w /= tiles_n;
  const uint32_t tm = w % tiles_m, z = w / tiles_m;
  return TileIndex{tm * TM, tn * TN, z % p.splits, z / p.splits};
}

// 256 threads, each a 4 x 4 block of the 64 x 64 tile.
__global__ void __launch_bounds__(256) gemm_f32_kernel(const GemmParams p) {
  __shared__ float As[kTK][kTM + 4];
  __shared__ float Bs[kTK][kTN + 4];
  grid_launch_dependents();   // launched with programmatic stream serialization, like the tensor kernels
  grid_dependency_wait();
  const uint32_t tid = threadIdx.x;
  const TileIndex tile = f32_tile_index<kTM, kTN>(p);
  const uint32_t split = tile.split, batch = tile.batch;
  const uint32_t m0 = tile.m0, n0 = tile.n0;
  const uint32_t k_begin = split * p.k_blocks_per_split * kTK;
  const uint32_t k_end = min(p.k, k_begin + p.k_blocks_per_split * kTK);
  const uint64_t a_off = (uint64_t)batch * p.ga.batch_stride, b_off = (uint64_t)batch * p.gbsrc.batch_stride;
  const uint32_t tr = tid / 16, tc = tid % 16;
  float acc[4][4] = {};
  for (uint32_t k0 = k_begin; k0 < k_end; k0 += kTK) {
    // A tile: 64 rows x 16 k.  K-major sources are contiguous along k, MN-major ones along m.
#pragma unroll
    for (uint32_t i = 0; i < 4; ++i) {
      const uint32_t e = tid + i * 256;
      uint32_t r, kk;
      if (p.ga.mn_major) { r = e % kTM; kk = e / kTM; } else { kk = e % kTK; r = e / kTK; }
      As[kk][r] = (k0 + kk < k_end) ? f32_operand(p.ga, p.geo, a_off, m0 + r, k0 + kk) : 0.0f;
    }
#pragma unroll
    for (uint32_t i = 0; i < 4; ++i) {
      const uint32_t e = tid + i * 256;
      uint32_t c, kk;
      if (p.gbsrc.mn_major) { c = e % kTN; kk = e / kTN; } else { kk = e % kTK; c = e / kTK; }
      Bs[kk][c] = (k0 + kk < k_end) ? f32_operand(p.gbsrc, p.geo, b_off, n0 + c, k0 + kk) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (uint32_t kk = 0; kk < kTK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (uint32_t i = 0; i < 4; ++i) a[i] = As[kk][tr * 4 + i];
#pragma unroll
      for (uint32_t j = 0; j < 4; ++j) b[j] = Bs[kk][tc * 4 + j];
#pragma unroll
      for (uint32_t i = 0; i < 4; ++i)
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (uint32_t i = 0; i < 4; ++i) {
    const uint32_t row = m0 + tr * 4 + i;
    if (row >= p.m) continue;
#pragma unroll
    for (uint32_t j = 0; j < 4; ++j) {
      const uint32_t col = n0 + tc * 4 + j;
      if (col >= p.n) continue;
      float x = acc[i][j];
      if (p.splits > 1) {
        p.partial[(((uint64_t)split * p.batch + batch) * p.m + row) * p.n + col] = x;
        continue;
      }
      const uint64_t idx = (uint64_t)batch * p.stride_c + (p.transpose_out ? (uint64_t)col * p.ldc + row : (uint64_t)row * p.ldc + col);
      if (p.accumulate) x += p.c_is_bf16 ? bf16_to_f32(((const uint16_t*)p.c)[idx]) : ((const float*)p.c)[idx];
      if (p.bias) x += p.bias[col];
      if (p.residual) x += p.c_is_bf16 ? bf16_to_f32(((const uint16_t*)p.residual)[idx]) : ((const float*)p.residual)[idx];
      if (p.relu) x = fmaxf(x, 0.0f);
      if (p.round_tf32) x = round_tf32(x);
      if (p.c_is_bf16) ((uint16_t*)p.c)[idx] = (uint16_t)bf16_bits(x);
      else ((float*)p.c)[idx] = x;
    }
  }
}

// ---- dense operands: the matmul family ----------------------------------------------------------------------
// Both operands are plain matrices, so nothing needs the per-element accessor above (a switch, 64-bit index
// arithmetic and bounds per element: ~2000 cycles per 16-deep K step, 16-18 TFLOP/s at best and 25-50 us for
// the MLP's one-tile products).  Each thread keeps pointers to its elements of the next K step and bumps them;
// the next step's elements are fetched into registers while the current step is multiplied out of shared
// memory.  TM x TN tile, 256 threads, (TM/16) x (TN/16) accumulators per thread.
template <int TM, int TN>
__global__ void __launch_bounds__(256) gemm_f32_dense_kernel(const GemmParams p) {
  constexpr int RM = TM / 16, RN = TN / 16, EA = TM * 16 / 256, EB = TN * 16 / 256;
  __shared__ __align__(16) float As[kTK][TM + 4];
  __shared__ __align__(16) float Bs[kTK][TN + 4];
  grid_launch_dependents();
  grid_dependency_wait();
  const uint32_t tid = threadIdx.x;
  const TileIndex tile = f32_tile_index<TM, TN>(p);
  const uint32_t split = tile.split, batch = tile.batch;
  const uint32_t m0 = tile.m0, n0 = tile.n0;
  const uint32_t k_begin = split * p.k_blocks_per_split * kTK;
  const uint32_t k_end = min(p.k, k_begin + p.k_blocks_per_split * kTK);
  // this thread's elements of a K step: (mn index within the tile, k index within the step), source pointer, row validity
  uint32_t a_r[EA], a_k[EA], b_c[EB], b_k[EB];
  int64_t a_off[EA], b_off[EB];
  bool a_ok[EA], b_ok[EB];
  const int64_t a_step = p.ga.mn_major ? (int64_t)kTK * p.ga.ld : kTK, b_step = p.gbsrc.mn_major ? (int64_t)kTK * p.gbsrc.ld : kTK;
#pragma unroll
  for (int i = 0; i < EA; ++i) {
    const uint32_t e = tid + i * 256;
    if (p.ga.mn_major) { a_r[i] = e % TM; a_k[i] = e / TM; } else { a_k[i] = e % kTK; a_r[i] = e / kTK; }
    const uint32_t row = m0 + a_r[i], kk = k_begin + a_k[i];
    a_ok[i] = row < p.m;
    a_off[i] = (int64_t)batch * p.ga.batch_stride + (p.ga.mn_major ? (int64_t)kk * p.ga.ld + row : (int64_t)row * p.ga.ld + kk);
  }
#pragma unroll
  for (int i = 0; i < EB; ++i) {
    const uint32_t e = tid + i * 256;
    if (p.gbsrc.mn_major) { b_c[i] = e % TN; b_k[i] = e / TN; } else { b_k[i] = e % kTK; b_c[i] = e / kTK; }
    const uint32_t col = n0 + b_c[i], kk = k_begin + b_k[i];
    b_ok[i] = col < p.n;
    b_off[i] = (int64_t)batch * p.gbsrc.batch_stride + (p.gbsrc.mn_major ? (int64_t)kk * p.gbsrc.ld + col : (int64_t)col * p.gbsrc.ld + kk);
  }
  auto fetch = [&](const GatherDesc& d, int64_t off) {
    return d.src_is_bf16 ? bf16_to_f32(((const uint16_t*)d.base)[off]) : ((const float*)d.base)[off];
  };
  float a_next[EA], b_next[EB];
  auto load_step = [&](uint32_t k0) {
#pragma unroll
    for (int i = 0; i < EA; ++i) {
      a_next[i] = (a_ok[i] && k0 + a_k[i] < k_end) ? fetch(p.ga, a_off[i]) : 0.0f;
      a_off[i] += a_step;
    }
#pragma unroll
    for (int i = 0; i < EB; ++i) {
      b_next[i] = (b_ok[i] && k0 + b_k[i] < k_end) ? fetch(p.gbsrc, b_off[i]) : 0.0f;
      b_off[i] += b_step;
    }
  };
  const uint32_t tr = tid / 16, tc = tid % 16;
  uint64_t acc2[RM][RN / 2];   // pairs of neighbouring columns
#pragma unroll
  for (int i = 0; i < RM; ++i)
#pragma unroll
    for (int j = 0; j < RN / 2; ++j) acc2[i][j] = 0ull;
  if (k_begin < k_end) load_step(k_begin);
  for (uint32_t k0 = k_begin; k0 < k_end; k0 += kTK) {
#pragma unroll
    for (int i = 0; i < EA; ++i) As[a_k[i]][a_r[i]] = a_next[i];
#pragma unroll
    for (int i = 0; i < EB; ++i) Bs[b_k[i]][b_c[i]] = b_next[i];
    __syncthreads();
    if (k0 + kTK < k_end) load_step(k0 + kTK);
#pragma unroll
    for (uint32_t kk = 0; kk < kTK; ++kk) {
      float a[RM];
      uint64_t b2[RN / 2];
#pragma unroll
      for (int i = 0; i < RM; i += 4) {
        const float4 v = *(const float4*)&As[kk][tr * RM + i];
        a[i] = v.x; a[i + 1] = v.y; a[i + 2] = v.z; a[i + 3] = v.w;
      }
#pragma unroll
      for (int j = 0; j < RN; j += 4) {
        const float4 v = *(const float4*)&Bs[kk][tc * RN + j];
        b2[j / 2] = pack_f32x2(v.x, v.y);
        b2[j / 2 + 1] = pack_f32x2(v.z, v.w);
      }
#pragma unroll
      for (int i = 0; i < RM; ++i) {
        const uint64_t aa = pack_f32x2(a[i], a[i]);
#pragma unroll
        for (int j = 0; j < RN / 2; ++j) acc2[i][j] = fma_f32x2(aa, b2[j], acc2[i][j]);
      }
    }
    __syncthreads();
  }
  float acc[RM][RN];
#pragma unroll
  for (int i = 0; i < RM; ++i)
#pragma unroll
    for (int j = 0; j < RN / 2; ++j) unpack_f32x2(acc2[i][j], acc[i][2 * j], acc[i][2 * j + 1]);
#pragma unroll
  for (int i = 0; i < RM; ++i) {
    const uint32_t row = m0 + tr * RM + i;
    if (row >= p.m) continue;
#pragma unroll
    for (int j = 0; j < RN; ++j) {
      const uint32_t col = n0 + tc * RN + j;
      if (col >= p.n) continue;
      float x = acc[i][j];
      if (p.splits > 1) {
        p.partial[(((uint64_t)split * p.batch + batch) * p.m + row) * p.n + col] = x;
        continue;
      }
      const uint64_t idx = (uint64_t)batch * p.stride_c + (p.transpose_out ? (uint64_t)col * p.ldc + row : (uint64_t)row * p.ldc + col);
      if (p.accumulate) x += p.c_is_bf16 ? bf16_to_f32(((const uint16_t*)p.c)[idx]) : ((const float*)p.c)[idx];
      if (p.bias) x += p.bias[col];
      if (p.residual) x += p.c_is_bf16 ? bf16_to_f32(((const uint16_t*)p.residual)[idx]) : ((const float*)p.residual)[idx];
      if (p.relu) x = fmaxf(x, 0.0f);
      if (p.round_tf32) x = round_tf32(x);
      if (p.c_is_bf16) ((uint16_t*)p.c)[idx] = (uint16_t)bf16_bits(x);
      else ((float*)p.c)[idx] = x;
    }
  }
}

}  // namespace

// Blocks of a strict-f32 launch with TM x TN tiles; 0 when the product is empty or does not fit grid.x.
uint32_t f32_grid_blocks(const GemmParams& p, uint32_t tm, uint32_t tn) {
  const uint64_t blocks = (uint64_t)((p.m + tm - 1) / tm) * ((p.n + tn - 1) / tn) * p.batch * p.splits;
  return blocks > 0x7FFFFFFFull ? 0u : (uint32_t)blocks;
}

// p.k_blocks_per_split counts blocks of 16 K values here.
cudaError_t launch_gemm_f32(const GemmParams& p, cudaStream_t stream) {
  if (p.m == 0 || p.n == 0 || p.batch == 0) return cudaSuccess;
  if (p.ga.source == kSrcDense && p.gbsrc.source == kSrcDense) {
    // 128 x 128 tiles once they fill the machine, 64 x 64 below that (more blocks, less work per block)
    const uint32_t big = f32_grid_blocks(p, 128, 128);
    if (big >= 148) {
      return launch_overlapped(gemm_f32_dense_kernel<128, 128>, dim3(big), dim3(256), 0, stream, p);
    } else {
      const uint32_t small = f32_grid_blocks(p, 64, 64);
      if (small == 0) return cudaErrorInvalidConfiguration;
      return launch_overlapped(gemm_f32_dense_kernel<64, 64>, dim3(small), dim3(256), 0, stream, p);
    }
  }
  const uint32_t blocks = f32_grid_blocks(p, kTM, kTN);
  if (blocks == 0) return cudaErrorInvalidConfiguration;
  return launch_overlapped(gemm_f32_kernel, dim3(blocks), dim3(256), 0, stream, p);
}

}  // namespace gb
