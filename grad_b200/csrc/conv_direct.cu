// Forward convolution of a layer with very few input channels (the 3-channel stem of ResNet-14: K = 3*3*3 = 27).
// Such a layer is no tensor-core shape: K fills less than half of one 64-wide K block, its input rows are 6 bytes
// apart (no TMA box can start there), and the gather warps of the contraction kernel spent ~12 us per 128-row
// tile building a mostly-zero operand tile -- a fifth of a whole ResNet-14 inference pass.  Here one thread
// owns four consecutive output positions and accumulates 16 output channels of each at a time with FMAs; the filters
// sit in shared memory as f32 and every lane reads the same 16 bytes of them (a broadcast).  The products are
// those of the tensor path: operands rounded to bf16 (GB_MATH_BF16) or to TF32 (GB_MATH_TF32), f32
// accumulation, then the same epilogue (old value, bias, residual, ReLU, rounding).  Follows the per-position
// definition in grad's src/gpu/math/conv.zig:47-65 (`patchOf`, `patchSource`) and :84-103 (forward).
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>

#include "gemm_sm100.cuh"
#include "sm100_ptx.cuh"

namespace gb {

namespace {

constexpr uint32_t kCoChunk = 16;   // output channels a thread accumulates at a time ...
constexpr uint32_t kPos = 4;        // ... for this many consecutive output positions

__device__ __forceinline__ float round_operand(float v, uint32_t tf32) {
  return tf32 ? round_tf32(v) : bf16_to_f32((uint16_t)bf16_bits(v));
}

// Dynamic shared memory: filters as f32 [taps * c][c_out], already rounded to the operand type, and behind them the
// patch values of the 128 positions a block works on, [taps * c][128] f32.  A block stages those once -- thread t fetches
// the taps * c values of position t, all loads independent -- and then every thread accumulates four consecutive
// positions x 16 channels from shared memory: per (tap, channel) one 16-byte read of patch values (the four lanes that
// hold the channel chunks of one position group read the same address) and four of filters feed 64 FMAs.  (Reading the
// patch values from global memory inside the FMA loop, 108 scattered 2-byte loads per thread, left the kernel waiting on
// them: 31 us for the stem at batch 128 against ~6 us of FMA time; with one position per thread it had been bound by the
// filter reads, 0.8 ms for 4096 images.)
constexpr uint32_t kTilePos = 128;

__global__ void __launch_bounds__(128) conv_direct_kernel(const GemmParams p) {
  extern __shared__ __align__(16) float w_s[];
  grid_launch_dependents();   // launched with programmatic stream serialization: wait for the stream's earlier work
  grid_dependency_wait();
  const ConvGeo& g = p.geo;
  const uint32_t kk = g.k * g.k * g.c;
  float* patch_s = w_s + ((kk * g.c_out + 3) & ~3u);
  for (uint32_t i = threadIdx.x; i < kk * g.c_out; i += blockDim.x) {
    const uint32_t row = i / g.c_out, co = i - row * g.c_out;
    const uint64_t idx = p.gbsrc.mn_major ? (uint64_t)row * p.gbsrc.ld + co : (uint64_t)co * p.gbsrc.ld + row;   // (K, c_out) or (c_out, K) rows
    const float v = p.gbsrc.src_is_bf16 ? bf16_to_f32(((const uint16_t*)p.gbsrc.base)[idx]) : ((const float*)p.gbsrc.base)[idx];
    w_s[i] = round_operand(v, p.tf32);
  }
  const uint32_t per_image = g.out_h * g.out_w;
  const uint32_t chunks = g.c_out / kCoChunk, tiles = (p.m + kTilePos - 1) / kTilePos;
  for (uint32_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    __syncthreads();   // the filters are in place; the previous tile's patch values are no longer read
    {
      // thread t stages position t of the tile (a position past the end repeats the last one and is not stored)
      const uint32_t pos = min(tile * kTilePos + threadIdx.x, p.m - 1);
      const uint32_t img = pos / per_image, rem = pos - img * per_image;
      const uint32_t oy = rem / g.out_w, ox = rem - oy * g.out_w;
      const uint32_t by = oy * g.stride, bx = ox * g.stride;
      uint32_t r = 0;
      for (uint32_t ky = 0; ky < g.k; ++ky)
        for (uint32_t kx = 0; kx < g.k; ++kx) {
          const uint32_t py = by + ky * g.dilation, px = bx + kx * g.dilation;
          const bool inside = py >= g.pad && py - g.pad < g.h && px >= g.pad && px - g.pad < g.w;
          const uint64_t src = inside ? ((uint64_t)(img * g.h + py - g.pad) * g.w + px - g.pad) * g.c_step : 0;
          for (uint32_t ci = 0; ci < g.c; ++ci, ++r) {
            float raw = 0.0f;
            if (inside) raw = p.ga.src_is_bf16 ? bf16_to_f32(((const uint16_t*)p.ga.base)[src + ci]) : round_operand(((const float*)p.ga.base)[src + ci], p.tf32);
            patch_s[r * kTilePos + threadIdx.x] = raw;
          }
        }
    }
    __syncthreads();
    // Work item = (group of kPos positions, chunk of kCoChunk channels), chunk fastest: neighbouring lanes hold the chunks
    // of one position group, so together they store whole 128-byte lines of the result and share their patch reads.
    for (uint32_t item = threadIdx.x; item < (kTilePos / kPos) * chunks; item += blockDim.x) {
      const uint32_t sub = item / chunks, co0 = (item - sub * chunks) * kCoChunk, grp = tile * (kTilePos / kPos) + sub;
      float acc[kPos][kCoChunk];
#pragma unroll
      for (uint32_t q = 0; q < kPos; ++q)
#pragma unroll
        for (uint32_t j = 0; j < kCoChunk; ++j) acc[q][j] = 0.0f;
#pragma unroll 3
      for (uint32_t r = 0; r < kk; ++r) {
        const float4 x4 = *(const float4*)(patch_s + r * kTilePos + sub * kPos);
        const float xv[kPos] = {x4.x, x4.y, x4.z, x4.w};
        const float4* w4 = (const float4*)(w_s + (uint64_t)r * g.c_out + co0);
#pragma unroll
        for (uint32_t j = 0; j < kCoChunk / 4; ++j) {
          const float4 wv = w4[j];
#pragma unroll
          for (uint32_t q = 0; q < kPos; ++q) {
            acc[q][4 * j] = fmaf(xv[q], wv.x, acc[q][4 * j]);
            acc[q][4 * j + 1] = fmaf(xv[q], wv.y, acc[q][4 * j + 1]);
            acc[q][4 * j + 2] = fmaf(xv[q], wv.z, acc[q][4 * j + 2]);
            acc[q][4 * j + 3] = fmaf(xv[q], wv.w, acc[q][4 * j + 3]);
          }
        }
      }
      float bias_r[kCoChunk];
#pragma unroll
      for (uint32_t j = 0; j < kCoChunk; ++j) bias_r[j] = p.bias ? p.bias[co0 + j] : 0.0f;
      // epilogue on 8 channels at a time: 16 bytes of bf16 or two 16-byte halves of f32
#pragma unroll
      for (uint32_t q = 0; q < kPos; ++q) {
        const uint32_t pos = grp * kPos + q;
        if (pos >= p.m) continue;
#pragma unroll
        for (uint32_t j = 0; j < kCoChunk; j += 8) {
          const uint64_t off = (uint64_t)pos * p.ldc + co0 + j;
          float v[8];
#pragma unroll
          for (uint32_t e = 0; e < 8; ++e) v[e] = acc[q][j + e];
          if (p.accumulate) {
            if (p.c_is_bf16) {
              const uint4 qq = *(const uint4*)((const uint16_t*)p.c + off);
              const uint32_t w[4] = {qq.x, qq.y, qq.z, qq.w};
#pragma unroll
              for (uint32_t e = 0; e < 4; ++e) { v[2 * e] += __uint_as_float(w[e] << 16); v[2 * e + 1] += __uint_as_float(w[e] & 0xFFFF0000u); }
            } else {
#pragma unroll
              for (uint32_t e = 0; e < 8; ++e) v[e] += ((const float*)p.c)[off + e];
            }
          }
#pragma unroll
          for (uint32_t e = 0; e < 8; ++e) v[e] += bias_r[j + e];
          if (p.residual) {
            if (p.c_is_bf16) {
              const uint4 qq = *(const uint4*)((const uint16_t*)p.residual + off);
              const uint32_t w[4] = {qq.x, qq.y, qq.z, qq.w};
#pragma unroll
              for (uint32_t e = 0; e < 4; ++e) { v[2 * e] += __uint_as_float(w[e] << 16); v[2 * e + 1] += __uint_as_float(w[e] & 0xFFFF0000u); }
            } else {
#pragma unroll
              for (uint32_t e = 0; e < 8; ++e) v[e] += ((const float*)p.residual)[off + e];
            }
          }
#pragma unroll
          for (uint32_t e = 0; e < 8; ++e) {
            if (p.relu) v[e] = fmaxf(v[e], 0.0f);
            if (p.round_tf32) v[e] = round_tf32(v[e]);
          }
          if (p.c_is_bf16) {
            *(uint4*)((uint16_t*)p.c + off) = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
          } else {
            *(float4*)((float*)p.c + off) = make_float4(v[0], v[1], v[2], v[3]);
            *(float4*)((float*)p.c + off + 4) = make_float4(v[4], v[5], v[6], v[7]);
          }
        }
      }
    }
  }
}

// ---- weight gradient of the same kind of layer --------------------------------------------------------------
// dw[(tap, ci), co] += sum over positions of patch(x)[pos, (tap, ci)] * dy[pos, co] with taps * c <= 36 rows (the stem:
// 27).  As a tensor-core product this has one 128-row tile that is four fifths padding, an A operand that only the
// gather warps can build, and K = all positions: 181 us for the stem at batch 128, a third of the whole network's
// weight-gradient time.  Here a block owns a contiguous range of positions and stages the patch values of 64 positions
// at a time in shared memory, with their dy rows (both rounded to the operand type like the tensor path; every global
// load of a tile is issued in that one staging phase, so their latencies overlap).  A thread keeps a 9-row x 4-channel
// block of partial sums in registers: its lanes split into (position, channel quad), its warp into a group of nine
// rows, so one 4-byte shared-memory read (two addresses per warp, different banks) feeds four FMAs.  (With one
// channel per thread every patch value was read once per FMA and the kernel was bound by those reads: 67 us.)
// Blocks write their partial matrices to the workspace and the split-K reduce kernel adds them in a fixed order, so
// the result does not depend on scheduling.
constexpr uint32_t kWgRows = 36;        // most (tap, channel) rows: four row groups of nine
constexpr uint32_t kWgRowsPerGroup = 9;
constexpr uint32_t kWgTile = 64;        // positions staged per round
constexpr uint32_t kWgThreads = 256;

__global__ void __launch_bounds__(kWgThreads) conv_direct_wgrad_kernel(const GemmParams p, uint32_t chunk) {
  __shared__ __align__(16) float patch_s[kWgTile][kWgRows];
  __shared__ float sum_s[kWgRows][64];
  __shared__ __align__(16) float dy_s[kWgTile][64];
  __shared__ int32_t row_dy[kWgRows], row_dx[kWgRows], row_ci[kWgRows];   // (tap, channel) row -> input offset and channel
  grid_launch_dependents();
  grid_dependency_wait();
  const ConvGeo& g = p.geo;
  const uint32_t rows = g.k * g.k * g.c, positions = p.k;
  const uint32_t span = min(g.c_out, 64u);             // output channels handled per pass
  const uint32_t quads = span / 4;                     // lanes per position: 4, 8, 16 or 32
  const uint32_t per_warp = 32 / quads;                // positions one warp instruction covers
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rg = warp & 3, pset = warp >> 2;      // row group; which half of the position slots
  const uint32_t quad = lane % quads, slot = pset * per_warp + lane / quads, slots = 2 * per_warp;
  const uint32_t per_image = g.out_h * g.out_w;
  const uint32_t begin = blockIdx.x * chunk, end = min(positions, begin + chunk);
  const bool dy_bf16 = p.gbsrc.src_is_bf16, x_bf16 = p.ga.src_is_bf16;
  if (threadIdx.x < kWgRows) {
    const uint32_t r = threadIdx.x, tap = r / g.c, ky = tap / g.k, kx = tap - ky * g.k;
    row_dy[r] = r < rows ? (int32_t)(ky * g.dilation) - (int32_t)g.pad : -(1 << 20);   // rows past the layer's read nothing
    row_dx[r] = (int32_t)(kx * g.dilation) - (int32_t)g.pad;
    row_ci[r] = (int32_t)(r - tap * g.c);
  }
  // staging role of this thread: one position of the tile, every fourth row of it
  const uint32_t st_pos = threadIdx.x % kWgTile, st_row0 = threadIdx.x / kWgTile;
  constexpr uint32_t kRowStep = kWgThreads / kWgTile;
  for (uint32_t co0 = 0; co0 < g.c_out; co0 += span) {
    const uint32_t co = co0 + quad * 4;
    float acc[kWgRowsPerGroup][4];
#pragma unroll
    for (uint32_t r = 0; r < kWgRowsPerGroup; ++r)
#pragma unroll
      for (uint32_t j = 0; j < 4; ++j) acc[r][j] = 0.0f;
    for (uint32_t t0 = begin; t0 < end; t0 += kWgTile) {
      __syncthreads();
      {
        // patch(x) of the tile's positions: this thread's position, every fourth row
        const uint32_t pos = t0 + st_pos;
        const bool valid = pos < end;
        const uint32_t img = pos / per_image, rem = pos - img * per_image, oy = rem / g.out_w, ox = rem - oy * g.out_w;
        const int32_t y0 = (int32_t)(oy * g.stride), x0 = (int32_t)(ox * g.stride);
#pragma unroll
        for (uint32_t r = st_row0; r < kWgRows; r += kRowStep) {
          const int32_t py = y0 + row_dy[r], px = x0 + row_dx[r];
          float v = 0.0f;
          if (valid && py >= 0 && px >= 0 && py < (int32_t)g.h && px < (int32_t)g.w) {
            const uint64_t idx = ((uint64_t)(img * g.h + py) * g.w + px) * g.c_step + row_ci[r];
            v = x_bf16 ? bf16_to_f32(((const uint16_t*)p.ga.base)[idx]) : round_operand(((const float*)p.ga.base)[idx], p.tf32);
          }
          patch_s[st_pos][r] = v;
        }
        // dy of the tile's positions x this pass's channels, as f32: coalesced 16-byte loads, all in flight together
        const uint32_t quads_per_row = span / 4;
        for (uint32_t e = threadIdx.x; e < kWgTile * quads_per_row; e += kWgThreads) {
          const uint32_t lp = e / quads_per_row, q4 = e - lp * quads_per_row, dpos = t0 + lp;
          float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
          if (dpos < end) {
            const uint64_t idx = (uint64_t)dpos * p.gbsrc.ld + co0 + q4 * 4;
            if (dy_bf16) {
              const uint2 raw = *(const uint2*)((const uint16_t*)p.gbsrc.base + idx);
              v = make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xFFFF0000u), __uint_as_float(raw.y << 16),
                              __uint_as_float(raw.y & 0xFFFF0000u));
            } else {
              const float4 raw = *(const float4*)((const float*)p.gbsrc.base + idx);
              v = make_float4(round_operand(raw.x, p.tf32), round_operand(raw.y, p.tf32), round_operand(raw.z, p.tf32), round_operand(raw.w, p.tf32));
            }
          }
          *(float4*)&dy_s[lp][q4 * 4] = v;
        }
      }
      __syncthreads();
      const uint32_t steps = kWgTile / slots;
#pragma unroll 4
      for (uint32_t st = 0; st < steps; ++st) {
        const uint32_t lp = st * slots + slot;
        const float4 dq = *(const float4*)&dy_s[lp][quad * 4];
        const float d[4] = {dq.x, dq.y, dq.z, dq.w};
        const float* prow = &patch_s[lp][rg * kWgRowsPerGroup];
#pragma unroll
        for (uint32_t r = 0; r < kWgRowsPerGroup; ++r) {
          const float v = prow[r];
#pragma unroll
          for (uint32_t j = 0; j < 4; ++j) acc[r][j] = fmaf(v, d[j], acc[r][j]);
        }
      }
    }
    // combine the position slots in slot order, then write this block's partial matrix [rows][c_out]
    for (uint32_t turn = 0; turn < slots; ++turn) {
      __syncthreads();
      if (slot == turn) {
#pragma unroll
        for (uint32_t r = 0; r < kWgRowsPerGroup; ++r)
#pragma unroll
          for (uint32_t j = 0; j < 4; ++j) {
            float* cell = &sum_s[rg * kWgRowsPerGroup + r][quad * 4 + j];
            *cell = turn == 0 ? acc[r][j] : *cell + acc[r][j];
          }
      }
    }
    __syncthreads();
    float* dst = p.partial + (uint64_t)blockIdx.x * rows * g.c_out;
    for (uint32_t e = threadIdx.x; e < rows * span; e += kWgThreads) {
      const uint32_t r = e / span, c = e - r * span;
      dst[(uint64_t)r * g.c_out + co0 + c] = sum_s[r][c];
    }
  }
}

}  // namespace

// Weight gradients this kernel takes: at most 36 (tap, channel) rows, 16, 32 or a multiple of 64 output channels,
// dy read as stored with 8-byte (bf16) or 16-byte (f32) aligned channel quads.
bool conv_direct_wgrad_applies(const GemmParams& p) {
  const ConvGeo& g = p.geo;
  const uint32_t rows = g.k * g.k * g.c;
  const bool lanes_ok = g.c_out == 16 || g.c_out == 32 || g.c_out % 64 == 0;
  const bool aligned = ((uintptr_t)p.gbsrc.base & 15) == 0 && p.gbsrc.ld % 4 == 0;
  return g.c <= 4 && rows <= kWgRows && lanes_ok && aligned && p.gbsrc.source == kSrcDense && p.ga.source == kSrcPatch && !p.transpose_out;
}
uint32_t conv_direct_wgrad_blocks(const GemmParams& p, int sm_count) {
  const uint32_t want = (p.k + 2 * kWgTile - 1) / (2 * kWgTile);      // at least two staged tiles per block
  return std::max(1u, std::min<uint32_t>(want, (uint32_t)sm_count * 4));
}
// `p.partial` holds blocks * rows * c_out floats; `p.splits` is set to the block count for the reduce launch that follows.
cudaError_t launch_conv_direct_wgrad(const GemmParams& p, uint32_t blocks, cudaStream_t stream) {
  if (p.k == 0) return cudaSuccess;
  const uint32_t chunk = (p.k + blocks - 1) / blocks;
  return launch_overlapped(conv_direct_wgrad_kernel, dim3(blocks), dim3(kWgThreads), 0, stream, p, chunk);
}

// The shapes this kernel takes: a forward pass whose whole filter fits 48 KB of shared memory as f32, output
// channels in whole chunks, and a result that can be stored 16 bytes at a time.
bool conv_direct_applies(const GemmParams& p) {
  const ConvGeo& g = p.geo;
  const uint64_t kk = (uint64_t)g.k * g.k * g.c;
  return g.c <= 4 && g.c_out % kCoChunk == 0 && (kk * g.c_out + kk * kTilePos + 4) * 4 <= 48 * 1024 && p.vec_store && !p.transpose_out;
}

cudaError_t launch_conv_direct(const GemmParams& p, int sm_count, cudaStream_t stream) {
  if (p.m == 0) return cudaSuccess;
  const ConvGeo& g = p.geo;
  const uint32_t kk = g.k * g.k * g.c;
  const size_t smem = (size_t)((kk * g.c_out + 3) & ~3u) * 4 + (size_t)kk * kTilePos * 4;   // filters, then one tile of patch values
  const uint32_t tiles = (p.m + kTilePos - 1) / kTilePos, cap = (uint32_t)sm_count * 4;
  return launch_overlapped(conv_direct_kernel, dim3(tiles < cap ? tiles : cap), dim3(128), smem, stream, p);
}

}  // namespace gb
