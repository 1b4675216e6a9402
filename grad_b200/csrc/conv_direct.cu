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

#include "gemm_sm100.cuh"
#include "sm100_ptx.cuh"

namespace gb {

namespace {

constexpr uint32_t kCoChunk = 16;   // output channels a thread accumulates at a time ...
constexpr uint32_t kPos = 4;        // ... for this many consecutive output positions

__device__ __forceinline__ float round_operand(float v, uint32_t tf32) {
  return tf32 ? round_tf32(v) : bf16_to_f32((uint16_t)bf16_bits(v));
}

// Dynamic shared memory: filters as f32 [taps * c][c_out], already rounded to the operand type.  A thread
// reads 16 bytes of them per four FMAs of ONE position; with one position per thread the kernel was bound
// by those shared-memory reads (0.8 ms for 4096 images), so a thread keeps four positions and every filter
// read feeds 16 FMAs.
__global__ void __launch_bounds__(128) conv_direct_kernel(const GemmParams p) {
  extern __shared__ float w_s[];
  grid_launch_dependents();   // launched with programmatic stream serialization: wait for the stream's earlier work
  grid_dependency_wait();
  const ConvGeo& g = p.geo;
  const uint32_t kk = g.k * g.k * g.c;
  for (uint32_t i = threadIdx.x; i < kk * g.c_out; i += blockDim.x) {
    const uint32_t row = i / g.c_out, co = i - row * g.c_out;
    const uint64_t idx = p.gbsrc.mn_major ? (uint64_t)row * p.gbsrc.ld + co : (uint64_t)co * p.gbsrc.ld + row;   // (K, c_out) or (c_out, K) rows
    const float v = p.gbsrc.src_is_bf16 ? bf16_to_f32(((const uint16_t*)p.gbsrc.base)[idx]) : ((const float*)p.gbsrc.base)[idx];
    w_s[i] = round_operand(v, p.tf32);
  }
  __syncthreads();
  const uint32_t per_image = g.out_h * g.out_w;
  // Work item = (group of kPos positions, chunk of kCoChunk channels), chunk fastest: neighbouring lanes hold
  // the chunks of one position group, so together they store whole 128-byte lines of the result and share
  // their input reads, and a small batch still yields enough threads to fill the machine.
  const uint32_t groups = (p.m + kPos - 1) / kPos, chunks = g.c_out / kCoChunk;
  const uint64_t items = (uint64_t)groups * chunks;
  for (uint64_t item = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; item < items; item += (uint64_t)gridDim.x * blockDim.x) {
    const uint32_t grp = (uint32_t)(item / chunks), co0 = (uint32_t)(item - (uint64_t)grp * chunks) * kCoChunk;
    // top-left input pixel (before padding is subtracted) and image of each of the thread's positions
    uint32_t base_y[kPos], base_x[kPos], image[kPos];
#pragma unroll
    for (uint32_t q = 0; q < kPos; ++q) {
      const uint32_t pos = min(grp * kPos + q, p.m - 1);   // a position past the end repeats the last one and is not stored
      const uint32_t img = pos / per_image, rem = pos - img * per_image;
      const uint32_t oy = rem / g.out_w;
      image[q] = img; base_y[q] = oy * g.stride; base_x[q] = (rem - oy * g.out_w) * g.stride;
    }
    {
      float acc[kPos][kCoChunk];
#pragma unroll
      for (uint32_t q = 0; q < kPos; ++q)
#pragma unroll
        for (uint32_t j = 0; j < kCoChunk; ++j) acc[q][j] = 0.0f;
      for (uint32_t ky = 0; ky < g.k; ++ky)
        for (uint32_t kx = 0; kx < g.k; ++kx) {
          int64_t src[kPos];
#pragma unroll
          for (uint32_t q = 0; q < kPos; ++q) {
            const uint32_t py = base_y[q] + ky * g.dilation, px = base_x[q] + kx * g.dilation;
            const bool inside = py >= g.pad && py - g.pad < g.h && px >= g.pad && px - g.pad < g.w;
            src[q] = inside ? (int64_t)(((uint64_t)(image[q] * g.h + py - g.pad) * g.w + px - g.pad) * g.c_step) : -1;
          }
          const float* wrow = w_s + (uint64_t)((ky * g.k + kx) * g.c) * g.c_out + co0;
          for (uint32_t ci = 0; ci < g.c; ++ci) {
            float xv[kPos];
#pragma unroll
            for (uint32_t q = 0; q < kPos; ++q) {
              float raw = 0.0f;
              if (src[q] >= 0) raw = p.ga.src_is_bf16 ? bf16_to_f32(((const uint16_t*)p.ga.base)[src[q] + ci]) : ((const float*)p.ga.base)[src[q] + ci];
              xv[q] = p.ga.src_is_bf16 ? raw : round_operand(raw, p.tf32);
            }
            const float4* w4 = (const float4*)(wrow + (uint64_t)ci * g.c_out);
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
        }
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
          if (p.bias) {
#pragma unroll
            for (uint32_t e = 0; e < 8; ++e) v[e] += p.bias[co0 + j + e];
          }
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

}  // namespace

// The shapes this kernel takes: a forward pass whose whole filter fits 48 KB of shared memory as f32, output
// channels in whole chunks, and a result that can be stored 16 bytes at a time.
bool conv_direct_applies(const GemmParams& p) {
  const ConvGeo& g = p.geo;
  const uint64_t kk = (uint64_t)g.k * g.k * g.c;
  return g.c <= 4 && g.c_out % kCoChunk == 0 && kk * g.c_out * 4 <= 48 * 1024 && p.vec_store && !p.transpose_out;
}

cudaError_t launch_conv_direct(const GemmParams& p, int sm_count, cudaStream_t stream) {
  if (p.m == 0) return cudaSuccess;
  const ConvGeo& g = p.geo;
  const size_t smem = (size_t)g.k * g.k * g.c * g.c_out * 4;
  const uint64_t items = (uint64_t)((p.m + kPos - 1) / kPos) * (g.c_out / kCoChunk);
  const uint64_t want64 = (items + 127) / 128;
  const uint32_t cap = (uint32_t)sm_count * 16, want = (uint32_t)(want64 < cap ? want64 : cap);
  return launch_overlapped(conv_direct_kernel, dim3(want < cap ? want : cap), dim3(128), smem, stream, p);
}

}  // namespace gb
