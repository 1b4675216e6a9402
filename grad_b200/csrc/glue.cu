// The few bandwidth-bound kernels the ONNX executor needs between contractions so that a whole ResNet graph
// stays on the device: 2-D pooling on NHWC, element-wise add / ReLU for node windows that were not folded
// into a convolution epilogue, dtype casts, and the OIHW -> (taps, c_out) weight reorder.  They follow the
// per-element definitions of grad's shared math (src/gpu/math/conv.zig:132-205 pooling,
// src/onnx/runtime.zig:845-862 `reorderOihw`); none of them is on the contraction path itself.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/gradb200.h"
#include "gemm_sm100.cuh"
#include "sm100_ptx.cuh"

namespace {

__device__ __forceinline__ float load_elem(const void* p, int bf16, size_t i) {
  return bf16 ? gb::bf16_to_f32(((const uint16_t*)p)[i]) : ((const float*)p)[i];
}
__device__ __forceinline__ void store_elem(void* p, int bf16, size_t i, float v) {
  if (bf16) ((uint16_t*)p)[i] = (uint16_t)gb::bf16_bits(v);
  else ((float*)p)[i] = v;
}

// Window clipped to the image like `boundsOf` (conv.zig:152-161); the average divides by the number of
// in-bounds taps (`windowCount`, :183-186).  One thread per output element.
__global__ void pool2d_kernel(const void* x, void* y, int bf16, int is_max, uint32_t n, uint32_t h, uint32_t w, uint32_t c, uint32_t k,
                              uint32_t stride, uint32_t pad, uint32_t oh, uint32_t ow) {
  const size_t total = (size_t)n * oh * ow * c;
  for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x) {
    const uint32_t ch = (uint32_t)(t % c), ox = (uint32_t)(t / c % ow), oy = (uint32_t)(t / c / ow % oh), img = (uint32_t)(t / c / ow / oh);
    const uint32_t top = oy * stride, left = ox * stride;
    const uint32_t y0 = top < pad ? 0 : top - pad, y1 = min(top + k - pad, h);
    const uint32_t x0 = left < pad ? 0 : left - pad, x1 = min(left + k - pad, w);
    float best = -INFINITY, sum = 0.0f;
    for (uint32_t yy = y0; yy < y1; ++yy)
      for (uint32_t xx = x0; xx < x1; ++xx) {
        const float v = load_elem(x, bf16, (((size_t)img * h + yy) * w + xx) * c + ch);
        best = fmaxf(best, v);
        sum += v;
      }
    const float count = (float)((y1 - y0) * (x1 - x0));
    store_elem(y, bf16, t, is_max ? best : sum / count);
  }
}

// The same pooling for bf16 tensors whose channel count is a multiple of 8: one thread per output pixel and
// group of 8 channels, 16-byte loads and stores, 32-bit index arithmetic.  (The scalar kernel above moved two
// bytes per thread behind four 64-bit divisions and reached an eighth of the memory bandwidth: 0.8 ms for
// the 537 MB activation of a 4096-image ResNet stage.)
__global__ void __launch_bounds__(256) pool2d_bf16x8_kernel(const uint4* x, uint4* y, int is_max, uint32_t n, uint32_t h, uint32_t w, uint32_t c8,
                                                            uint32_t k, uint32_t stride, uint32_t pad, uint32_t oh, uint32_t ow) {
  gb::grid_launch_dependents();   // launched with programmatic stream serialization: wait for the stream's earlier work
  gb::grid_dependency_wait();
  const uint32_t total = n * oh * ow * c8;   // the caller keeps this below 2^32
  for (uint32_t t = blockIdx.x * blockDim.x + threadIdx.x; t < total; t += gridDim.x * blockDim.x) {
    const uint32_t pix = t / c8, cg = t - pix * c8;
    const uint32_t row = pix / ow, ox = pix - row * ow;
    const uint32_t img = row / oh, oy = row - img * oh;
    const uint32_t top = oy * stride, left = ox * stride;
    const uint32_t y0 = top < pad ? 0 : top - pad, y1 = min(top + k - pad, h);
    const uint32_t x0 = left < pad ? 0 : left - pad, x1 = min(left + k - pad, w);
    float acc[8];
#pragma unroll
    for (uint32_t e = 0; e < 8; ++e) acc[e] = is_max ? -INFINITY : 0.0f;
    for (uint32_t yy = y0; yy < y1; ++yy) {
      const uint4* line = x + ((size_t)(img * h + yy) * w) * c8 + cg;
      for (uint32_t xx = x0; xx < x1; ++xx) {
        const uint4 q = line[(size_t)xx * c8];
        const uint32_t wd[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (uint32_t e = 0; e < 4; ++e) {
          const float lo = __uint_as_float(wd[e] << 16), hi = __uint_as_float(wd[e] & 0xFFFF0000u);
          acc[2 * e] = is_max ? fmaxf(acc[2 * e], lo) : acc[2 * e] + lo;
          acc[2 * e + 1] = is_max ? fmaxf(acc[2 * e + 1], hi) : acc[2 * e + 1] + hi;
        }
      }
    }
    if (!is_max) {
      const float count = (float)((y1 - y0) * (x1 - x0));
#pragma unroll
      for (uint32_t e = 0; e < 8; ++e) acc[e] = acc[e] / count;
    }
    y[t] = make_uint4(gb::pack_bf16x2(acc[0], acc[1]), gb::pack_bf16x2(acc[2], acc[3]), gb::pack_bf16x2(acc[4], acc[5]), gb::pack_bf16x2(acc[6], acc[7]));
  }
}

// op 0: out = a + b; 1: out = relu(a); 2: out = relu(a + b); 3: out = a + bias[i % cols] (b is f32 bias)
__global__ void elementwise_kernel(const void* a, const void* b, void* out, int bf16, int op, size_t total, uint32_t cols) {
  for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x) {
    float v = load_elem(a, bf16, t);
    if (op == 0 || op == 2) v += load_elem(b, bf16, t);
    if (op == 3) v += ((const float*)b)[t % cols];
    if (op == 1 || op == 2) v = fmaxf(v, 0.0f);
    store_elem(out, bf16, t, v);
  }
}

__global__ void cast_kernel(const void* src, void* dst, int src_bf16, int dst_bf16, size_t total) {
  for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x)
    store_elem(dst, dst_bf16, t, load_elem(src, src_bf16, t));
}

// w is (m, c, kh, kw) f32; wt is (kh*kw*c, m): wt[(tap*c + ic)*m + oc] = w[(oc*c + ic)*khkw + tap].
__global__ void reorder_oihw_kernel(const float* w, void* wt, int dst_bf16, uint32_t m, uint32_t c, uint32_t khkw) {
  const size_t total = (size_t)m * c * khkw;
  for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x) {
    const uint32_t oc = (uint32_t)(t % m);
    const size_t item = t / m;
    const uint32_t ic = (uint32_t)(item % c), tap = (uint32_t)(item / c);
    store_elem(wt, dst_bf16, t, w[((size_t)oc * c + ic) * khkw + tap]);
  }
}

// wt is (m, kh*kw*c): wt[oc*(khkw*c) + tap*c + ic] = w[(oc*c + ic)*khkw + tap].
__global__ void reorder_oihw_rows_kernel(const float* w, void* wt, int dst_bf16, uint32_t m, uint32_t c, uint32_t khkw) {
  const size_t total = (size_t)m * c * khkw;
  for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x) {
    const uint32_t ic = (uint32_t)(t % c), tap = (uint32_t)(t / c % khkw), oc = (uint32_t)(t / c / khkw);
    store_elem(wt, dst_bf16, t, w[((size_t)oc * c + ic) * khkw + tap]);
  }
}

// (n, c, h, w) <-> (n, h, w, c) for graphs that arrive in NCHW (src/onnx/gpu.zig:525-542).
__global__ void permute_kernel(const void* src, void* dst, int bf16, int to_nhwc, uint32_t n, uint32_t c, uint32_t h, uint32_t w) {
  const size_t total = (size_t)n * c * h * w;
  for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x) {
    // t indexes the destination
    size_t s;
    if (to_nhwc) {
      const uint32_t ch = (uint32_t)(t % c), x = (uint32_t)(t / c % w), y = (uint32_t)(t / c / w % h), img = (uint32_t)(t / c / w / h);
      s = (((size_t)img * c + ch) * h + y) * w + x;
    } else {
      const uint32_t x = (uint32_t)(t % w), y = (uint32_t)(t / w % h), ch = (uint32_t)(t / w / h % c), img = (uint32_t)(t / w / h / c);
      s = (((size_t)img * h + y) * w + x) * c + ch;
    }
    store_elem(dst, bf16, t, load_elem(src, bf16, s));
  }
}

unsigned blocks_for(size_t total) {
  const size_t want = (total + 255) / 256;
  return (unsigned)(want < 148 * 8 ? (want == 0 ? 1 : want) : 148 * 8);
}

int finish() { return cudaGetLastError() == cudaSuccess ? GB_OK : GB_ERR_CUDA; }



// (rows, cols) f32 -> (cols, rows) in the destination type through a 32 x 33 shared-memory tile: both sides coalesced.
__global__ void transpose_cast_kernel(const float* src, void* dst, int dst_bf16, uint32_t rows, uint32_t cols) {
  __shared__ float tile[32][33];
  const uint32_t r0 = blockIdx.y * 32, c0 = blockIdx.x * 32;
  for (uint32_t i = threadIdx.y; i < 32; i += blockDim.y) {
    const uint32_t r = r0 + i, c = c0 + threadIdx.x;
    tile[i][threadIdx.x] = (r < rows && c < cols) ? src[(size_t)r * cols + c] : 0.0f;
  }
  __syncthreads();
  for (uint32_t i = threadIdx.y; i < 32; i += blockDim.y) {
    const uint32_t c = c0 + i, r = r0 + threadIdx.x;
    if (c < cols && r < rows) store_elem(dst, dst_bf16, (size_t)c * rows + r, tile[threadIdx.x][i]);
  }
}

}  // namespace

// A prepared copy of one f32 master weight matrix: where it came from, where the copy lives, how to remake it.
struct gb_weights {
  const float* master;
  void* data;
  uint32_t rows, cols;
  int kind, dtype;
};

namespace {

int convert_weights(const gb_weights* w, cudaStream_t stream) {
  const size_t total = (size_t)w->rows * w->cols;
  if (total == 0) return GB_OK;
  if (w->kind == GB_WEIGHTS_PLAIN) return gb_cast(stream, GB_F32, w->dtype, w->master, w->data, total);
  const dim3 grid((w->cols + 31) / 32, (w->rows + 31) / 32), block(32, 8);
  transpose_cast_kernel<<<grid, block, 0, stream>>>(w->master, w->data, w->dtype == GB_BF16, w->rows, w->cols);
  return cudaGetLastError() == cudaSuccess ? GB_OK : GB_ERR_CUDA;
}

}  // namespace

namespace {
// s = gamma * inv_std and t = beta - mean * s per channel, each rounded to bf16 (`affineExpand`, src/gpu/device.zig:1774-1783).
__global__ void affine_expand_kernel(const float* mean, const float* inv_std, const float* gamma, const float* beta, uint16_t* scale,
                                     uint16_t* shift, uint32_t c) {
  const uint32_t ch = blockIdx.x * blockDim.x + threadIdx.x;
  if (ch >= c) return;
  const float s = __fmul_rn(gamma[ch], inv_std[ch]);
  scale[ch] = (uint16_t)gb::bf16_bits(s);
  shift[ch] = (uint16_t)gb::bf16_bits(__fsub_rn(beta[ch], __fmul_rn(mean[ch], s)));
}
}  // namespace

namespace gb {
cudaError_t launch_affine_expand(const float* mean, const float* inv_std, const float* gamma, const float* beta, uint16_t* scale, uint16_t* shift,
                                 uint32_t c, cudaStream_t stream) {
  affine_expand_kernel<<<(c + 127) / 128, 128, 0, stream>>>(mean, inv_std, gamma, beta, scale, shift, c);
  return cudaGetLastError();
}
}  // namespace gb

extern "C" {

size_t gb_weights_bytes(uint32_t rows, uint32_t cols, int dtype) { return (size_t)rows * cols * (dtype == GB_BF16 ? 2 : 4); }

int gb_prepare_weights(void* stream, const float* master, uint32_t rows, uint32_t cols, int kind, int dtype, void* storage, size_t storage_bytes,
                       gb_weights** out) {
  if (!out) return GB_ERR_INVALID;
  *out = nullptr;
  if (!master || !storage || (kind != GB_WEIGHTS_PLAIN && kind != GB_WEIGHTS_ROWS) || (dtype != GB_F32 && dtype != GB_BF16)) return GB_ERR_INVALID;
  if (storage_bytes < gb_weights_bytes(rows, cols, dtype) || ((uintptr_t)storage & 15) != 0) return GB_ERR_INVALID;
  gb_weights* w = new gb_weights{master, storage, rows, cols, kind, dtype};
  const int rc = convert_weights(w, (cudaStream_t)stream);
  if (rc != GB_OK) {
    delete w;
    return rc;
  }
  *out = w;
  return GB_OK;
}

int gb_refresh_weights(const gb_weights* weights, void* stream) { return weights ? convert_weights(weights, (cudaStream_t)stream) : GB_ERR_INVALID; }
const void* gb_weights_data(const gb_weights* weights) { return weights ? weights->data : nullptr; }
void gb_weights_destroy(gb_weights* weights) { delete weights; }

int gb_pool2d(void* stream, int is_max, int dtype, const void* x, void* y, uint32_t n, uint32_t h, uint32_t w, uint32_t c, uint32_t k,
              uint32_t stride, uint32_t pad) {
  if (!x || !y || k == 0 || stride == 0 || h + 2 * pad < k || w + 2 * pad < k) return GB_ERR_INVALID;
  const uint32_t oh = (h + 2 * pad - k) / stride + 1, ow = (w + 2 * pad - k) / stride + 1;
  const size_t total = (size_t)n * oh * ow * c;
  if (total == 0) return GB_OK;
  if (dtype == GB_BF16 && c % 8 == 0 && total / 8 < 0xFFFFFFFFull && ((uintptr_t)x & 15) == 0 && ((uintptr_t)y & 15) == 0) {
    const size_t groups = total / 8;
    const size_t want = (groups + 255) / 256;
    const cudaError_t e = gb::launch_overlapped(pool2d_bf16x8_kernel, dim3((unsigned)(want < 148 * 16 ? want : 148 * 16)), dim3(256), 0, (cudaStream_t)stream,
                                                (const uint4*)x, (uint4*)y, is_max, n, h, w, c / 8, k, stride, pad, oh, ow);
    return e == cudaSuccess ? GB_OK : GB_ERR_CUDA;
  }
  pool2d_kernel<<<blocks_for(total), 256, 0, (cudaStream_t)stream>>>(x, y, dtype == GB_BF16, is_max, n, h, w, c, k, stride, pad, oh, ow);
  return finish();
}

int gb_elementwise(void* stream, int op, int dtype, const void* a, const void* b, void* out, size_t total, uint32_t cols) {
  if (!a || !out || op < 0 || op > 3 || ((op == 0 || op == 2 || op == 3) && !b) || (op == 3 && cols == 0)) return GB_ERR_INVALID;
  if (total == 0) return GB_OK;
  elementwise_kernel<<<blocks_for(total), 256, 0, (cudaStream_t)stream>>>(a, b, out, dtype == GB_BF16, op, total, cols);
  return finish();
}

int gb_cast(void* stream, int src_dtype, int dst_dtype, const void* src, void* dst, size_t total) {
  if (!src || !dst) return GB_ERR_INVALID;
  if (total == 0) return GB_OK;
  cast_kernel<<<blocks_for(total), 256, 0, (cudaStream_t)stream>>>(src, dst, src_dtype == GB_BF16, dst_dtype == GB_BF16, total);
  return finish();
}

int gb_reorder_oihw(void* stream, int dst_dtype, const float* w, void* wt, uint32_t m, uint32_t c, uint32_t kh, uint32_t kw) {
  if (!w || !wt) return GB_ERR_INVALID;
  const size_t total = (size_t)m * c * kh * kw;
  if (total == 0) return GB_OK;
  reorder_oihw_kernel<<<blocks_for(total), 256, 0, (cudaStream_t)stream>>>(w, wt, dst_dtype == GB_BF16, m, c, kh * kw);
  return finish();
}

int gb_reorder_oihw_rows(void* stream, int dst_dtype, const float* w, void* wt, uint32_t m, uint32_t c, uint32_t kh, uint32_t kw) {
  if (!w || !wt) return GB_ERR_INVALID;
  const size_t total = (size_t)m * c * kh * kw;
  if (total == 0) return GB_OK;
  reorder_oihw_rows_kernel<<<blocks_for(total), 256, 0, (cudaStream_t)stream>>>(w, wt, dst_dtype == GB_BF16, m, c, kh * kw);
  return finish();
}

int gb_permute_layout(void* stream, int dtype, int to_nhwc, const void* src, void* dst, uint32_t n, uint32_t c, uint32_t h, uint32_t w) {
  if (!src || !dst) return GB_ERR_INVALID;
  const size_t total = (size_t)n * c * h * w;
  if (total == 0) return GB_OK;
  permute_kernel<<<blocks_for(total), 256, 0, (cudaStream_t)stream>>>(src, dst, dtype == GB_BF16, to_nhwc, n, c, h, w);
  return finish();
}

}  // extern "C"
