/*
 * CPU oracle for the dense-contraction path of hyunjun3952/grad.
 *
 * TEST INFRASTRUCTURE ONLY.  This library restates, in plain C++, the arithmetic of the
 * reference's CPU backend (the backend its own tests compare the GPU against).  It is the
 * checker for the CUDA kernels and the timed CPU baseline of the benchmark; the product
 * library never links, loads or calls it.
 *
 * Parity status: PINNED.  The reference is Zig and cannot be built here, so the pin is the
 * reference's own known-answer tests and exact-equality properties, re-run against this
 * restatement by tests/test_oracle_golden.py (tests/tensor.zig:34-42,93-103;
 * tests/kernels.zig:13-148; tests/bf16.zig:7-14; tests/runtime.zig:66-84;
 * tests/cpu_ops.zig:14-117; tests/autograd.zig:702-733).
 *
 * Every function cites the reference file:line it follows.
 */
#ifndef GRAD_ORACLE_H
#define GRAD_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* src/gpu/math/conv.zig:22 `Dims` (same field order, all u32). */
typedef struct {
  uint32_t n, h, w, c, k, stride, pad, dilation, groups, c_out;
} oracle_dims;

/* src/gpu/math/bf16.zig:1-5 and :39-41. */
uint16_t oracle_bf16_encode(float x);
float oracle_bf16_decode(uint16_t h);
void oracle_bf16_round_array(const float* src, float* dst, size_t n);   /* decode(encode(x)) */
void oracle_bf16_encode_array(const float* src, uint16_t* dst, size_t n);
void oracle_bf16_decode_array(const uint16_t* src, float* dst, size_t n);
/* src/gpu/device.zig:1888-1893: cvt.rna.tf32.f32 (round to nearest, ties away, 10-bit mantissa). */
float oracle_tf32_round(float x);
void oracle_tf32_round_array(const float* src, float* dst, size_t n);

/* src/cpu/kernels.zig:20-32 `matmulNaive`: acc += a*b with separate multiply and add. */
void oracle_matmul_naive_f32(size_t m, size_t k, size_t n, const float* a, const float* b, float* out);
void oracle_matmul_naive_f64(size_t m, size_t k, size_t n, const double* a, const double* b, double* out);

/* src/cpu/kernels.zig:234-448 `splitFor` + `matmulTiled` + `matmulTiledRange`, default TileConfig
 * (mr 6, nv 2, mc 96, kc 256, nc 1024).  `threads` <= 1 means a Parallel without a pool (one part).
 * `kc_override`/`mc_override`/`nc_override` of 0 keep the defaults (tests/kernels.zig uses a second
 * TileConfig).  Stored layouts: a is (m,k), or (k,m) when trans_a; b is (k,n), or (n,k) when trans_b. */
void oracle_matmul_tiled_f32(size_t m, size_t k, size_t n, const float* a, const float* b, float* out,
                             int trans_a, int trans_b, int accumulate, int threads);
void oracle_matmul_tiled_f64(size_t m, size_t k, size_t n, const double* a, const double* b, double* out,
                             int trans_a, int trans_b, int accumulate, int threads);
void oracle_matmul_tiled_cfg_f32(size_t m, size_t k, size_t n, const float* a, const float* b, float* out,
                                 int trans_a, int trans_b, int accumulate, int threads,
                                 size_t mr, size_t nv, size_t mc, size_t kc, size_t nc);
/* Which axis splitFor picks: 0 rows, 1 cols, 2 depth; *parts and *chunk receive the split. */
int oracle_split_for(size_t m, size_t k, size_t n, int threads, size_t* parts, size_t* chunk);

/* src/gpu/math/conv.zig:24-30. */
uint32_t oracle_out_height(const oracle_dims* d);
uint32_t oracle_out_width(const oracle_dims* d);
/* src/gpu/math/conv.zig:71-84 per-element im2col / :104-131 per-element col2im (dx += ...). */
void oracle_im2col_elements(const float* x, float* col, const oracle_dims* d);
void oracle_col2im_elements(const float* dcol, float* dx, const oracle_dims* d);
/* src/cpu/ops.zig:12-53 row-wise im2col with the memcpy fast path, :253-285 col2im per pixel. */
void oracle_im2col_rows(const float* x, float* col, const oracle_dims* d, size_t first, size_t count, int threads);
void oracle_col2im_pixels(const float* dcol, float* dx, const oracle_dims* d, int threads);

/* src/cpu/ops.zig:131-148 `convForward` (chunked im2col x matmulTiled, direct single-channel path :84-129). */
void oracle_conv_forward(const float* x, const float* w, float* out, const oracle_dims* d, int threads);
/* src/cpu/ops.zig:152-170 `convInputGrad` (dx += col2im(grad * w^T)). */
void oracle_conv_input_grad(const float* grad, const float* w, float* dx, const oracle_dims* d, int threads);
/* src/cpu/ops.zig:235-251 `convWeightGrad` (dw += im2col(x)^T * grad; direct path :172-231). */
void oracle_conv_weight_grad(const float* x, const float* grad, float* dw, const oracle_dims* d, int threads);
/* src/gpu/math/conv.zig:259-340 grouped convolution, per element (forward stores, grads add). */
void oracle_conv_grouped_forward(const float* x, const float* w, float* out, const oracle_dims* d);
void oracle_conv_grouped_input_grad(const float* dy, const float* w, float* dx, const oracle_dims* d);
void oracle_conv_grouped_weight_grad(const float* x, const float* dy, float* dw, const oracle_dims* d);
/* tests/autograd.zig:702-733: the 7-loop direct convolution in f64, an independent cross-check. */
void oracle_conv_direct_f64(const float* x, const float* w, double* out, const oracle_dims* d);

/* src/onnx/runtime.zig:845-862 `reorderOihw`: (m,c,kh,kw) -> (kh*kw*c, m). */
void oracle_reorder_oihw(const float* w, float* wt, size_t m, size_t c, size_t kh, size_t kw);
/* src/onnx/runtime.zig:868-899 `convolveNhwc` (+ `addBias(.nhwc)` :714-742); w is OIHW. bias may be NULL. */
void oracle_convolve_nhwc(const float* x, const float* w_oihw, const float* bias, float* out,
                          const oracle_dims* d, int threads);
/* src/onnx/runtime.zig:755-838 `convolve` on NCHW with groups (group-free: planar im2col x matmulTiled). */
void oracle_convolve_nchw(const float* x, const float* w_oihw, const float* bias, float* out,
                          size_t n, size_t c, size_t h, size_t width, size_t m, size_t kh, size_t kw,
                          size_t groups, size_t stride, size_t pad, size_t dilation, int threads);
/* src/onnx/runtime.zig:621-646 `matmul` (batched; weight batch 1 broadcasts) and :648-664 `gemm`. */
void oracle_onnx_matmul(const float* x, const float* y, float* out, size_t batch, size_t weight_batch,
                        size_t m, size_t k, size_t n, int threads);
void oracle_onnx_gemm(const float* x, const float* y, const float* c, float* out, size_t m, size_t k, size_t n,
                      int trans_a, int trans_b, float alpha, float beta, int threads);
/* src/onnx/runtime.zig:515-517 Relu. */
void oracle_relu(float* v, size_t n);
/* The unfused sequence that defines a fused epilogue (src/autograd/autograd.zig:449-468,
 * src/onnx/gpu.zig:518-519, 372-377): out[r][c] = act(out[r][c] + bias[c]), in f32. */
void oracle_bias_act(float* out, const float* bias, size_t rows, size_t cols, int relu);

/* src/nn/replicas.zig:57-91 `averageGrads`: mean over replicas, summed in replica order, then
 * scaled by 1/N; every replica receives the same bits. grads is replicas x len, updated in place. */
void oracle_average_grads(float* grads, size_t replicas, size_t len);

/* Host facts for the benchmark line. */
int oracle_host_threads(void);
int oracle_vector_lanes(void);   /* f32 lanes of the micro-tile in use: 16 (AVX-512), 8 (AVX2) or 8 scalar */

#ifdef __cplusplus
}
#endif
#endif
