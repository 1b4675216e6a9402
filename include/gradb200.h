/*
 * gradb200.h -- C ABI of libgradb200.so: the dense-contraction path of hyunjun3952/grad
 * (matmul family + implicit-GEMM conv2d + gradient allreduce) as hand-written sm_100a kernels.
 *
 * The library is loaded the way grad loads libcuda and cuDNN: dlopen + one dlsym per entry point
 * into a struct of C function pointers (src/gpu/dynlib.zig:20-61, src/gpu/cudnn.zig:22-86,120-127).
 * Conventions, taken from the callers in src/gpu/gpu.zig:
 *   - every pointer argument is a raw device address from cuMemAlloc (gpu.zig:395-410); the library
 *     never frees, retains or allocates tensors.  bf16 is uint16_t storage (src/gpu/math/bf16.zig).
 *   - temporaries come from a caller-owned workspace (like cudnn_workspace, gpu.zig:485-501); the
 *     size is asked with the *_workspace query.  No entry point allocates device memory after
 *     gb_create, none synchronises, none reads back: all are safe under stream capture
 *     (src/gpu/cuda.zig:151-159).
 *   - `stream` is the CUstream the caller launches on (NULL = legacy default stream, cuda.zig:210-212).
 *   - return value: 0 on success, a gb_status otherwise (cuda.zig:118-124); never aborts or throws.
 *   - there is no CPU fallback: without a CUDA device every compute entry point fails.
 */
#ifndef GRADB200_H
#define GRADB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GB_ABI_VERSION 3

typedef struct gb_handle gb_handle;   /* per-device state; one per host thread, like one `Gpu` per thread */
typedef struct gb_comm gb_comm;       /* one rank of a gradient-averaging group */

typedef enum {
  GB_OK = 0,
  GB_ERR_INVALID = 1,       /* bad argument (null pointer, zero stride, trans_a and trans_b both set, ...) */
  GB_ERR_CUDA = 2,          /* a CUDA call failed; gb_last_cuda_error() has the code (maps to error.CudaFailed) */
  GB_ERR_WORKSPACE = 3,     /* gb_gemm_static_scratch: the partial sums exceed the fixed array; ordered batch-norm statistics
                             * without room for their partials (error.OutOfMemory).  Otherwise gb_gemm and gb_conv_* do not
                             * return it: with a workspace that is null, misaligned or smaller than the *_workspace query said,
                             * they run the product unsplit (and gather f32 master filters) instead */
  GB_ERR_UNSUPPORTED = 4,   /* shape / dtype combination outside what the kernels cover (error.NoAlgorithm) */
  GB_ERR_TIMEOUT = 5,       /* a bounded wait gave up: on the device (see gb_last_status) or for a peer replica (gb_comm_*) */
  GB_ERR_NCCL = 6,          /* NCCL missing or a collective failed */
  GB_ERR_NO_DEVICE = 7      /* no CUDA device / not an sm_100 part (error.NoSuchDevice) */
} gb_status;

typedef enum { GB_F32 = 0, GB_BF16 = 1 } gb_dtype;

/* Arithmetic of the contraction.  Accumulation is always f32.
 *   GB_MATH_F32  strict f32 FMA on the CUDA cores (device.zig `f32Compute` :1665-1684, `Gemm` :122-201)
 *   GB_MATH_TF32 operands read as TF32 by the tensor core (`tf32Compute` :1888-1913)
 *   GB_MATH_BF16 operands rounded to bf16 (RNE) when not already bf16 (`bf16Compute` :997-1045) */
typedef enum { GB_MATH_F32 = 0, GB_MATH_TF32 = 1, GB_MATH_BF16 = 2 } gb_math;

typedef enum { GB_ACT_NONE = 0, GB_ACT_RELU = 1 } gb_activation;

/* Fused epilogue.  grad has no fused bias today: `Tape.linear` adds the bias with a second launch
 * (src/autograd/autograd.zig:449-468) and the ONNX executor adds bias and applies Relu with two more
 * (src/onnx/gpu.zig:518-519, 372-377).  The fused result is defined as that unfused sequence in f32:
 *   v = acc (+ old C when accumulate) ; v += bias[col] ; v += residual[row][col] ; v = act(v) ; store. */
/* Batch-norm statistics summed in the epilogue, the role of `BnStats` / `statsTile` (src/gpu/device.zig:1447, 1505-1535;
 * host side `Gpu.convImplicitForwardStats`, src/gpu/gpu.zig:915-923): for every output column (channel) the sums of
 * (v - shift[col]) and of (v - shift[col])^2 over all rows (positions), taken over the values AS STORED (rounded to bf16
 * when the result is bf16), are ADDED to sums[col] and sums[n + col]; the caller zeroes `sums` (`scratchZeroed`).  shift is
 * the running mean, a close estimate that keeps the squared sums precise.  The stored result is bit-identical to the
 * same call without statistics (tests/gpu.zig:205): the statistics plan adds up K in the order the plain plan of the same
 * call uses (it cannot follow a plain plan that splits K: a product of a few row tiles with K >= 2048).  ordered = 1 is the reference's deterministic mode: every CTA writes
 * its partial sums to the workspace and a second launch adds them in a fixed order, so repeated runs give identical
 * bits; ordered = 0 adds with atomics.  Needs n <= 256, n a multiple of 32 and a 16-byte aligned row-major result
 * (every ResNet training layer); otherwise the call returns GB_ERR_UNSUPPORTED and nothing is launched. */
typedef struct {
  const float* shift;       /* f32[n] */
  float* sums;              /* f32[2 * n]: += */
  uint32_t ordered;
  uint32_t reserved;
} gb_bn_stats;

/* The sums a batch-norm backward needs, from the epilogue of the input-gradient product whose result is the gradient with
 * respect to a normalised-and-rectified map that was never written (`DxStats` / `dxStatsTile`, src/gpu/device.zig:1452,
 * 1537-1580; `Gpu.convImplicitForwardDxStats`, src/gpu/gpu.zig:964-972): x is the raw bf16 map the norm ran on, laid out
 * like dx; x_hat = (x - mean) * inv_std; where gamma * x_hat + beta > 0 the stored gradient g counts, elsewhere it is 0;
 * sums[col] += sum g, sums[n + col] += sum g * x_hat.  dx itself is stored unmasked.  Same shape limits and `ordered`
 * meaning as gb_bn_stats; dx must be bf16. */
typedef struct {
  const void* x;            /* bf16, same shape and pitch as dx */
  const float *mean, *inv_std, *gamma, *beta;   /* f32[n] each */
  float* sums;              /* f32[2 * n]: += */
  uint32_t ordered;
  uint32_t reserved;
} gb_dx_stats;

typedef struct {
  const float* bias;        /* f32[n] (per output column / output channel) or NULL */
  const void* residual;     /* same shape, pitch and dtype as the output, or NULL (ONNX Add before Relu) */
  int32_t activation;       /* gb_activation */
  int32_t flags;            /* GB_EPILOGUE_* bits */
  const gb_bn_stats* bn_stats;   /* NULL, or per-column statistics of the stored result (see gb_bn_stats) */
} gb_epilogue;
/* Round the stored f32 result to TF32 (nearest, ties away: cvt.rna.tf32.f32, src/gpu/device.zig:1888-1893).
 * The tensor core reads TF32 operands by dropping the low mantissa bits; a chain of TF32 layers whose
 * activations were rounded when stored sees the reference's round-to-nearest instead of a truncation. */
#define GB_EPILOGUE_ROUND_TF32 1

/* One product C[m,n] (+)= op(A) * op(B), row-major.  Replaces `MatmulShape` + `MatmulOpts`
 * (src/gpu/gpu.zig:22,29), `GemmShape` (src/gpu/args.zig:2-12) and the fields of `TensorShape`
 * (args.zig:72) that `Gpu.matmulPacked` sets (gpu.zig:1036-1064).
 *   trans_a: A is stored (k, m);  trans_b: B is stored (n, k);  never both (gpu.zig:643).
 *   lda/ldb/ldc: row pitch in elements of the STORED matrices; 0 = dense (the stored row length).
 *   batch > 1: that many consecutive products, operands stride_* elements apart (args.zig:1-12);
 *              a stride of 0 broadcasts that operand.
 *   batch_outer > 1: a second batch level: product (o, i), i < batch, o < batch_outer, reads and writes at
 *              i * stride_x + o * stride_x_outer.  For operands whose batch entries are not equally spaced: the heads
 *              of a (rows, heads * width) activation, one product per (sequence, head) of an attention layer in one
 *              launch.  Tensor-core path with both operands reachable by TMA only (16-byte aligned strides), no K
 *              split; otherwise GB_ERR_UNSUPPORTED.
 *   transpose_out: C is written as (n, m) with pitch ldc (args.zig `transpose_out`).
 *   deterministic: split-K partials are combined in a fixed order (gpu.zig:1024-1034); this
 *              library's split-K is always ordered, so the flag only documents the caller's intent. */
typedef struct {
  uint32_t m, n, k, batch;
  uint64_t stride_a, stride_b, stride_c;
  uint32_t lda, ldb, ldc;
  uint8_t trans_a, trans_b, accumulate, transpose_out;
  uint8_t dtype_a, dtype_b, dtype_c, math;   /* gb_dtype x3, gb_math */
  uint8_t deterministic, reserved[3];
  uint32_t batch_outer, reserved2;            /* 0 or 1: a single batch level */
  uint64_t stride_a_outer, stride_b_outer, stride_c_outer;
} gb_gemm_desc;

/* Field-for-field copy of `ConvGeometry` (src/gpu/args.zig:78) so a Zig `extern struct` passes by
 * pointer.  Always the FORWARD geometry of the layer: x is (n,h,w,c) NHWC, y is (n,out_h,out_w,c_out),
 * w is (k*k*c, c_out) with row (ky*k+kx)*c+ci (src/autograd/autograd.zig:91,1150).  positions =
 * n*out_h*out_w.  c_step = channel stride of x in memory (0 = c).  subsample is ignored: the input
 * gradient entry point derives the reverse gather itself instead of taking a reversed geometry and
 * rotated weights (autograd.zig:101-125, gpu.zig:856-866). */
typedef struct {
  uint32_t n, h, w, c, k, stride, pad, out_h, out_w, positions, c_out, dilation, c_step, subsample;
} gb_conv_geometry;

typedef struct {
  gb_conv_geometry geo;
  uint8_t dtype_x, dtype_w, dtype_y, math;   /* dtype of x (or dx), of w (or dw), of y (or dy); gb_math */
  uint8_t accumulate, deterministic;
  uint8_t w_layout;          /* 0: w is (k*k*c, c_out) as grad stores it; 1 (forward only): w is (c_out, k*k*c), a copy
                              * prepared once per weight -- the role of the executor's `reorderedWeights` cache
                              * (src/onnx/gpu.zig:566-574).  With K contiguous per output channel two CTAs can
                              * split even a 64-channel filter bank, so 256 positions share one MMA. */
  uint8_t reserved;
  uint32_t groups;           /* 0 or 1: dense.  > 1: grouped convolution (src/gpu/math/conv.zig:259-340): input channels
                              * [g*c/groups, (g+1)*c/groups) feed output channels [g*c_out/groups, ...); w is (k*k*c/groups, c_out)
                              * with row (ky*k+kx)*(c/groups)+ic.  Runs as one product per group over channel slices of x, w and y,
                              * the reference's `grouped_implicit` path (src/autograd/autograd.zig:150-155, 1041, 1129); plain
                              * layers only (w_layout 0, no statistics). */
} gb_conv_desc;

/* ---- lifetime --------------------------------------------------------------------------------- */
/* Uses the primary context of `device_ordinal` like `Cuda.init` (src/gpu/cuda.zig:67-83); created in
 * `Gpu.init`, destroyed in `Gpu.deinit` (src/gpu/gpu.zig:362-392).  Allocates one status word. */
int gb_create(int device_ordinal, gb_handle** out);
void gb_destroy(gb_handle* h);
int gb_abi_version(void);
const char* gb_error_string(int status);
/* Last cudaError_t seen by this handle (0 if none). */
int gb_last_cuda_error(const gb_handle* h);
/* Reads (and clears) the device-side status word: 0 = every bounded wait completed.  Synchronises the
 * stream, so call it outside capture -- the analogue of `Gpu.sync` + error check. */
int gb_last_status(gb_handle* h, void* stream, uint32_t* device_status);
/* Multiprocessor count the tile/split heuristics use (src/gpu/gpu.zig `multiprocessors`). */
int gb_sm_count(const gb_handle* h);

/* How the last gb_gemm / gb_conv_* call on this handle was cut up -- the counterpart of reading
 * `gemmTile`, `splits` and `forwardPlan` in src/gpu/gpu.zig:659-697, 890-913 when profiling.
 * operand kinds: 0 TMA K-major tile, 1 TMA MN-major tile, 2 TMA NHWC patch box (K-major), 3 TMA NHWC
 * patch box (MN-major, weight gradient), 4 TMA weight box (input gradient), 5 gathered with plain loads. */
typedef struct {
  uint32_t tensor_path;     /* 1 = tcgen05 kernel, 0 = strict-f32 CUDA-core kernel */
  uint32_t a_kind, b_kind;
  uint32_t tile_m, tile_n, stages, splits, k_blocks, work_items, kernel_launches;
} gb_plan_info;
int gb_last_plan(const gb_handle* h, gb_plan_info* out);
/* A handle keeps the prepared plans (tile choice, tensor maps) of its recent calls, keyed by descriptor, addresses,
 * epilogue and workspace, so that a repeated call -- every step of a training loop, every pass of the executor --
 * costs the host a key compare and a launch instead of ~15 us of planning.  Returns how many calls were served from
 * that cache so far (GB_NO_PLAN_CACHE in the environment turns it off). */
uint64_t gb_plan_cache_hits(const gb_handle* h);

/* ---- matmul family ---------------------------------------------------------------------------- */
/* Replaces `Gpu.matmul` (src/gpu/gpu.zig:642-679), `Gpu.matmulTensor` / `packMatrix` / `matmulPacked`
 * (:1066-1073, :711-722, :1036-1064) and the kernels `sgemm*` / `sgemmTensor`
 * (src/gpu/device.zig:122-250, 1710-1712).  Operands are consumed in place: no packed copies. */
int gb_gemm_workspace(const gb_handle* h, const gb_gemm_desc* desc, size_t* bytes);
int gb_gemm(gb_handle* h, void* stream, const gb_gemm_desc* desc, const void* a, const void* b, void* c,
            const gb_epilogue* epilogue, void* workspace, size_t workspace_bytes);

/* gb_gemm for callers that cannot allocate device memory (no counterpart in the reference, whose callers
 * always own an arena: src/gpu/gpu.zig:395-410).  It takes no handle -- gb_create allocates -- and no
 * workspace: split-K partial sums go to a fixed GB_STATIC_SCRATCH_BYTES array inside the library image,
 * held by every GPU that loads the library until the process exits.  It uses the CURRENT device.  The
 * first call with a given device current resolves the array's device address; make that call outside
 * stream capture.  A product whose partials exceed the array returns GB_ERR_WORKSPACE.  All calls share
 * the array: calls that overlap on the GPU (two streams, two threads) race and must be serialised.
 * A bounded device-side wait that gave up leaves C partly written; gb_static_last_status (the handle-free
 * gb_last_status: synchronises the stream, reads and clears a status word that also lives in the library image)
 * then returns GB_ERR_TIMEOUT.  It allocates nothing either. */
#define GB_STATIC_SCRATCH_BYTES (4u << 20)
int gb_gemm_static_scratch(void* stream, const gb_gemm_desc* desc, const void* a, const void* b, void* c,
                           const gb_epilogue* epilogue);
int gb_static_last_status(void* stream, uint32_t* device_status);

/* ---- implicit-GEMM convolution ---------------------------------------------------------------- */
/* Forward: replaces `Gpu.convImplicitForward` (src/gpu/gpu.zig:926-929), `Gpu.convF32Forward`
 * (:789-826), the im2col+GEMM paths `chooseConvPath` picks for strided or narrow layers
 * (src/autograd/autograd.zig:143-163) and `Executor.convNhwc` (src/onnx/gpu.zig:576-610).
 * y[n,oy,ox,co] (+)= sum x[n, oy*s+ky*d-p, ox*s+kx*d-p, ci] * w[(ky*k+kx)*c+ci, co], then the epilogue. */
int gb_conv_workspace(const gb_handle* h, int pass /*0 fprop, 1 dgrad, 2 wgrad*/, const gb_conv_desc* desc, size_t* bytes);
int gb_conv_fprop(gb_handle* h, void* stream, const gb_conv_desc* desc, const void* x, const void* w, void* y,
                  const gb_epilogue* epilogue, void* workspace, size_t workspace_bytes);
/* Forward pass over an input that stands for a batch norm + ReLU of the stored map x that was never written out:
 * every in-bounds tap reads relu(s * x + t) with s = gamma * inv_std and t = beta - mean * s per input channel, both
 * rounded to bf16 and applied as one bf16 fused multiply-add (`affineExpand` / `affinePair`, src/gpu/device.zig:1774-1805,
 * 1604-1612); padding taps stay exactly zero.  Replaces `Gpu.convImplicitForwardAffineStats` (src/gpu/gpu.zig:951-959;
 * the statistics part is `epilogue->bn_stats`).  bf16 activations and bf16 math only.  Where TMA can fetch the map (channel
 * counts in multiples of 64, up to 2048) it arrives with NaN outside the image and two warps rewrite each landed tile in shared memory
 * before the tensor core reads it (NaN -> 0: the reference's marker trick, device.zig:77-86), 1.4-2 times the time of
 * gb_conv_fprop; otherwise the gather warps transform while they build the tile, far slower.  The first 4 * c bytes of the
 * workspace (rounded up to 256) are reserved for the expanded s and t: the gather path fills them with one extra launch,
 * the TMA path expands the norm inside the kernel (a table in shared memory) and leaves them untouched. */
typedef struct {
  const float *mean, *inv_std, *gamma, *beta;   /* f32[c] each: the norm that the input stands for */
} gb_affine_input;
int gb_conv_fprop_affine(gb_handle* h, void* stream, const gb_conv_desc* desc, const void* x, const void* w, void* y,
                         const gb_epilogue* epilogue, const gb_affine_input* affine, void* workspace, size_t workspace_bytes);
/* Input gradient: dx (+)= conv_transpose(dy, w).  Replaces `convImplicitForward` / `convF32Forward` on
 * the reversed geometry with `packRotatedWeights` / `rotateWeightsF32` (gpu.zig:754-772, 856-866) and
 * the `*Subsampled` kernels for strided layers (device.zig:1921-1925). */
int gb_conv_dgrad(gb_handle* h, void* stream, const gb_conv_desc* desc, const void* dy, const void* w, void* dx,
                  void* workspace, size_t workspace_bytes);
/* The same product with the batch-norm backward sums of gb_dx_stats in its epilogue (stride-1 layers, dx stored, not
 * accumulated): `Gpu.convImplicitForwardDxStats`. */
int gb_conv_dgrad_stats(gb_handle* h, void* stream, const gb_conv_desc* desc, const void* dy, const void* w, void* dx,
                        const gb_dx_stats* stats, void* workspace, size_t workspace_bytes);
/* Weight gradient: dw[(tap,ci),co] (+)= sum_positions patch(x)[pos,(tap,ci)] * dy[pos,co], f32 output.
 * Replaces `Gpu.convImplicitWeightGrad` (gpu.zig:983-1022) and `convF32WeightGrad` + `transposeF32`
 * (:775-787, :828-866).  Partials of the split over positions are combined in order. */
int gb_conv_wgrad(gb_handle* h, void* stream, const gb_conv_desc* desc, const void* dy, const void* x, void* dw,
                  void* workspace, size_t workspace_bytes);
/* The weight gradient over the same kind of virtual input (the `...Affine` weight-gradient kernels,
 * src/gpu/device.zig:1756-1766; `convImplicitWeightGrad(..., aff)`, src/gpu/gpu.zig:983-1022). */
int gb_conv_wgrad_affine(gb_handle* h, void* stream, const gb_conv_desc* desc, const void* dy, const void* x, void* dw,
                         const gb_affine_input* affine, void* workspace, size_t workspace_bytes);

/* ---- prepared weights -------------------------------------------------------------------------- */
/* grad keeps f32 master weights and converts them on EVERY use: `packMatrix` before each forward product and
 * `packRotatedWeights` before each input gradient (src/autograd/autograd.zig:955, 967, 1226, 1272, 1345, 1350, 1401,
 * 1418; src/gpu/gpu.zig:711-722).  With a prepared copy the conversion happens once per optimizer step instead: the
 * caller makes the copy after `adam.step` (src/nn/optim.zig:122-150) with gb_refresh_weights and passes
 * gb_weights_data() as `w` (dtype_w = the copy's dtype) to gb_gemm / gb_conv_fprop / gb_conv_dgrad, which then fetch
 * every operand by TMA and launch no cast.  No rotated copy exists or is needed: gb_conv_dgrad reads the forward
 * layout.  The copy lives in caller-owned device memory (`storage`, gb_weights_bytes() bytes, 16-byte aligned): the
 * library allocates nothing on the device; the gb_weights object is a few host words.
 *   GB_WEIGHTS_PLAIN  the master's (rows, cols) layout -- (k*k*c_in, c_out) filters, (n_in, n_out) Linear weights
 *   GB_WEIGHTS_ROWS   transposed to (cols, rows): filters as (c_out, k*k*c_in) for gb_conv_desc.w_layout = 1, or a
 *                     Linear weight as the K-major B operand of `trans_b` */
typedef struct gb_weights gb_weights;
typedef enum { GB_WEIGHTS_PLAIN = 0, GB_WEIGHTS_ROWS = 1 } gb_weights_kind;
size_t gb_weights_bytes(uint32_t rows, uint32_t cols, int dtype);
int gb_prepare_weights(void* stream, const float* master_f32, uint32_t rows, uint32_t cols, int kind, int dtype, void* storage,
                       size_t storage_bytes, gb_weights** out);
/* Remakes the copy from the master (one launch on `stream`, capture-safe): call it after the optimizer step. */
int gb_refresh_weights(const gb_weights* weights, void* stream);
const void* gb_weights_data(const gb_weights* weights);
void gb_weights_destroy(gb_weights* weights);

/* ---- executor glue (ONNX inference graphs) ------------------------------------------------------ */
/* The bandwidth-bound node kinds `grad.onnx_gpu.Executor` runs between contractions, so a ResNet graph
 * never leaves the device (src/onnx/gpu.zig:304-470): all take the caller's stream, none allocates.
 * dtype is a gb_dtype; tensors are NHWC. */
/* MaxPool / AveragePool with a square window; windows are clipped to the image and the average divides by
 * the in-bounds count (src/gpu/math/conv.zig:152-205). */
int gb_pool2d(void* stream, int is_max, int dtype, const void* x, void* y, uint32_t n, uint32_t h, uint32_t w, uint32_t c,
              uint32_t k, uint32_t stride, uint32_t pad);
/* op 0: out = a + b; 1: out = relu(a); 2: out = relu(a + b); 3: out = a + bias[i % cols] with b an f32 bias
 * (`elementwise(.add)` + `Relu`, src/onnx/gpu.zig:318, 372-377, 518-519). */
int gb_elementwise(void* stream, int op, int dtype, const void* a, const void* b, void* out, size_t total, uint32_t cols);
int gb_cast(void* stream, int src_dtype, int dst_dtype, const void* src, void* dst, size_t total);
/* OIHW f32 filters -> (kh*kw*c, m) in dst_dtype: `reorderedWeights` / `reorderOihw`
 * (src/onnx/gpu.zig:566-574, src/onnx/runtime.zig:845-862); done once per weight and cached by the caller. */
int gb_reorder_oihw(void* stream, int dst_dtype, const float* w, void* wt, uint32_t m, uint32_t c, uint32_t kh, uint32_t kw);
/* The same filters as (m, kh*kw*c): layout 1 of gb_conv_desc.w_layout. */
int gb_reorder_oihw_rows(void* stream, int dst_dtype, const float* w, void* wt, uint32_t m, uint32_t c, uint32_t kh, uint32_t kw);
/* NCHW <-> NHWC copy for graphs that arrive in NCHW (src/onnx/gpu.zig:525-542). */
int gb_permute_layout(void* stream, int dtype, int to_nhwc, const void* src, void* dst, uint32_t n, uint32_t c, uint32_t h, uint32_t w);

/* ---- data-parallel gradient mean -------------------------------------------------------------- */
/* Replaces `Replicas.averageGrads` (src/nn/replicas.zig:57-91): the mean over replicas of ONE flat f32
 * gradient vector (`gradLen`, replicas.zig:95-99), in place, identical bits on every rank -- one NCCL
 * allreduce over NVLink instead of two trips through host memory.  unique_id is 128 bytes from
 * gb_comm_unique_id on rank 0, shared by the caller.  device_ordinal < 0 keeps the current device.
 * The communicator is non-blocking and every wait has a host deadline (gb_comm_set_timeout, default 60 s or
 * GB_COMM_TIMEOUT_MS): a replica that never joins makes gb_comm_create / gb_allreduce_mean / gb_comm_finish
 * abort the communicator and return GB_ERR_TIMEOUT, the counterpart of `Replicas.stop` releasing the waiters
 * with error.Stopped (replicas.zig:36-53).  After an abort every call on the communicator returns GB_ERR_NCCL. */
int gb_comm_unique_id(void* out128);
int gb_comm_create(int nranks, int rank, const void* unique_id128, int device_ordinal, gb_comm** out);
int gb_comm_set_timeout(gb_comm* comm, uint32_t timeout_ms);
/* Enqueues the mean on `stream` and returns (capture-safe once the communicator exists). */
int gb_allreduce_mean(gb_comm* comm, void* stream, float* grads, size_t count);
/* Host-side wait for `stream` with the communicator's deadline: GB_OK when the work on the stream has finished;
 * when the deadline passes first, the communicator is aborted (which ends a collective still waiting for a peer
 * on the device) and GB_ERR_TIMEOUT is returned.  The bounded form of the barrier after the reduction
 * (replicas.zig:81). */
int gb_comm_finish(gb_comm* comm, void* stream);
int gb_comm_abort(gb_comm* comm);     /* the analogue of `Replicas.stop` (replicas.zig:36-38) */
void gb_comm_destroy(gb_comm* comm);

#ifdef __cplusplus
}
#endif
#endif /* GRADB200_H */
