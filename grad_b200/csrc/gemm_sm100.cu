// The tcgen05 contraction kernel: one persistent, warp-specialised CTA per SM computes 128 x BN output
// tiles of C = A * B with f32 accumulators in tensor memory.
//
//   warp 0      TMA producer: every box of a stage has its own lane, which keeps the box's four coordinates in
//               registers and steps them from K block to K block with the same instructions in every lane; the
//               stage's "full" mbarrier counts the bytes.
//   warp 1      MMA issuer: owns the TMEM allocation; one thread (chosen by elect.sync) issues four tcgen05.mma
//               per K block (K = 16 bf16 or 8 tf32 each) from descriptors built once per kernel -- several K
//               blocks per stage for column-patch convolution stages and weight gradients -- and commits the
//               stage's "empty" barrier; after the last K block of a tile it commits the accumulator's "full"
//               barrier.  Both loops poll the next stage's barrier one iteration ahead of its use.
//   warps 2-9   epilogue, two warps per 32-lane quarter of TMEM (they split the column chunks): tcgen05.ld
//               double-buffered in registers, accumulator handed back as soon as the last read has landed,
//               (+C) (+bias from shared memory) (+residual) (ReLU), rounding to the output type, then a 32 x 64
//               byte block staged in shared memory and written by a TMA store (per-lane 16-byte stores for
//               transposed, ragged, mapped or split-K results).  Two accumulator buffers let the epilogue of
//               tile i overlap the mainloop of tile i+1.
//   warps 10-11 (only when an operand cannot be fetched by TMA) gather warps fill the stage with plain
//               loads: any pitch, f32 -> bf16 conversion on the fly, implicit im2col of NHWC activations
//               for any stride / dilation / padding / channel count.
//
// The prologue (barriers by warp 2, TMEM by warp 1, the producer's box set-up by warp 0, cluster sync) touches no global
// memory; launched with programmatic stream serialization it overlaps the tail of the previous kernel in the stream, and
// each role executes griddepcontrol.wait only right before its first global access.
//
// The same kernel serves the dense matmul family (NN / NT / TN through K-major or MN-major shared-memory
// descriptors, no packed or transposed copies) and the implicit-GEMM convolutions (forward, input
// gradient, weight gradient) whose activation operand is fetched as 4-D TMA boxes of the NHWC tensor.
// Replaces grad's `tileGemm` (src/gpu/device.zig:1162-1708) and `Gemm` (:122-201) tensor paths.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "gemm_sm100.cuh"
#include "sm100_ptx.cuh"

namespace gb {

namespace {

constexpr uint32_t kBM = 128;            // tile rows = TMEM lanes
constexpr uint32_t kLineBytes = 128;     // one swizzled line
constexpr uint32_t kATileBytes = kBM * kLineBytes;
constexpr uint32_t kMaxStages = 8;
constexpr uint32_t kHeaderBytes = 1024;  // barriers + TMEM base + abort flag, ahead of the 1024-aligned tiles

struct SmemHeader {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t xfull[kMaxStages];   // transformed-operand plans: the stage's A tile has been rewritten in place
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t spin_limit;   // directly behind abort_flag: the bounded waits read it as abort_flag[1]
};

struct Work {
  uint32_t batch, m_tile, n_tile, split, kb_begin, kb_end;
  uint32_t empty;   // fused classes: this tile lies past the rows of its class; every role skips it
};

__device__ __forceinline__ uint32_t fast_div(uint32_t a, const FastDiv& f) {
  uint32_t q = __umulhi(a, f.m);
  uint32_t r = a - q * f.d;
  if (r >= f.d) { r -= f.d; ++q; }
  if (r >= f.d) { ++q; }
  return q;
}

// Work item -> tile.  Every role of a CTA decodes every item, and a short-K tile (a convolution layer is 9-36 K
// blocks) is over in a few thousand cycles, so the common shapes skip the divisions: no K split, one batch
// entry, one column of tiles.
__device__ __forceinline__ Work decode_work(const GemmParams& p, uint32_t w) {
  Work out;
  uint32_t t = w;
  out.split = 0;
  if (p.splits > 1) {
    t = fast_div(w, p.div_splits);
    out.split = w - t * p.splits;
  }
  out.batch = 0;
  if (p.batch > 1) {
    out.batch = fast_div(t, p.div_per_batch);
    t -= out.batch * p.div_per_batch.d;
  }
  if (p.tiles_n == 1) {
    out.m_tile = t;
    out.n_tile = 0;
  } else {
    const uint32_t band = fast_div(t, p.div_band);
    const uint32_t within = t - band * p.div_band.d;
    const uint32_t rows_in_band = min(p.group_m, p.tiles_m - band * p.group_m);
    out.n_tile = rows_in_band == p.group_m ? fast_div(within, p.div_group) : within / rows_in_band;   // only the last band is shorter
    out.m_tile = band * p.group_m + within - out.n_tile * rows_in_band;
  }
  out.kb_begin = out.split * p.k_blocks_per_split;
  out.kb_end = min(out.kb_begin + p.k_blocks_per_split, p.k_blocks_total);
  out.empty = 0;
  if (p.n_classes) {
    out.kb_end = p.cls[out.batch].k_blocks;
    out.empty = out.m_tile * (p.cta_pair ? 2 * kBM : kBM) >= p.cls[out.batch].m;
  }
  return out;
}

// Two batch levels: work item b -> (inner, outer) indices, and where its C matrix starts.
__device__ __forceinline__ void split_batch(const GemmParams& p, uint32_t batch, uint32_t& inner, uint32_t& outer) {
  inner = batch;
  outer = 0;
  if (p.batch_inner) {
    outer = fast_div(batch, p.div_batch_inner);
    inner = batch - outer * p.batch_inner;
  }
}
__device__ __forceinline__ uint64_t c_batch_offset(const GemmParams& p, uint32_t batch) {
  uint32_t inner, outer;
  split_batch(p, batch, inner, outer);
  return (uint64_t)inner * p.stride_c + (uint64_t)outer * p.stride_c_outer;
}

// ---- gather sources ---------------------------------------------------------------------------------

__device__ __forceinline__ float load_as_f32(const GatherDesc& d, int64_t idx) {
  if (idx < 0) return 0.0f;
  return d.src_is_bf16 ? bf16_to_f32(((const uint16_t*)d.base)[idx]) : ((const float*)d.base)[idx];
}

// What a gathered line needs from its line-major index, computed once per line instead of once per element.
struct LineCtx {
  uint32_t line, valid;
  uint32_t img;
  int32_t y0, x0;   // patch: top-left input coordinate of the window (may be negative); patchT: pixel + pad
};

__device__ __forceinline__ LineCtx make_line_ctx(const GatherDesc& d, const ConvGeo& g, uint32_t line) {
  LineCtx c;
  c.line = line;
  c.valid = line < d.lines_total;
  c.img = 0; c.y0 = 0; c.x0 = 0;
  if (!c.valid) return c;
  if (d.source == kSrcPatch) {
    const uint32_t per_image = g.out_h * g.out_w;
    c.img = line / per_image;
    const uint32_t rem = line - c.img * per_image, oy = rem / g.out_w, ox = rem - oy * g.out_w;
    c.y0 = (int32_t)(oy * g.stride) - (int32_t)g.pad;
    c.x0 = (int32_t)(ox * g.stride) - (int32_t)g.pad;
  } else if (d.source == kSrcPatchT) {
    const uint32_t per_image = g.h * g.w;
    c.img = line / per_image;
    const uint32_t rem = line - c.img * per_image, y = rem / g.w, x = rem - y * g.w;
    c.y0 = (int32_t)(y + g.pad);
    c.x0 = (int32_t)(x + g.pad);
  }
  return c;
}

// Source index of element `inner` of the line, or -1 for an implicit zero; `run` receives how many elements
// from there on are contiguous in memory and share that answer (capped at `want`).
__device__ __forceinline__ int64_t gather_run(const GatherDesc& d, const ConvGeo& g, const LineCtx& c, uint32_t inner, uint32_t want, uint32_t& run) {
  run = want;
  if (!c.valid || inner >= d.inner_total) return -1;
  run = min(want, d.inner_total - inner);
  switch (d.source) {
    case kSrcDense:
      return (int64_t)c.line * d.ld + inner;
    case kSrcPatch: {
      const uint32_t tap = inner / g.c, ci = inner - tap * g.c;
      const uint32_t ky = tap / g.k, kx = tap - ky * g.k;
      run = min(run, g.c - ci);
      const int32_t py = c.y0 + (int32_t)(ky * g.dilation), px = c.x0 + (int32_t)(kx * g.dilation);
      if (py < 0 || px < 0 || py >= (int32_t)g.h || px >= (int32_t)g.w) return -1;
      return ((int64_t)(c.img * g.h + py) * g.w + px) * g.c_step + ci;
    }
    case kSrcPatchT: {
      const uint32_t tap = inner / g.c_out, co = inner - tap * g.c_out;
      const uint32_t ky = tap / g.k, kx = tap - ky * g.k;
      run = min(run, g.c_out - co);
      const int32_t ty = c.y0 - (int32_t)(ky * g.dilation), tx = c.x0 - (int32_t)(kx * g.dilation);
      if (ty < 0 || tx < 0) return -1;
      const uint32_t oy = (uint32_t)ty / g.stride, ox = (uint32_t)tx / g.stride;
      if (oy * g.stride != (uint32_t)ty || ox * g.stride != (uint32_t)tx || oy >= g.out_h || ox >= g.out_w) return -1;
      return ((int64_t)(c.img * g.out_h + oy) * g.out_w + ox) * g.y_step + co;
    }
    default: {
      const uint32_t tap = inner / g.c_out, co = inner - tap * g.c_out;
      run = min(run, g.c_out - co);
      return ((int64_t)tap * g.c + c.line) * g.w_step + co;
    }
  }
}

// Fills one 128-byte line of an operand tile.  `l` is the line's index within the tile (its low bits select
// the swizzle).  All eight 16-byte chunks are fetched before any is stored, so their latencies overlap;
// a chunk that is one aligned contiguous run (or all padding) takes vector loads, anything else goes
// element by element.
__device__ __forceinline__ void gather_line(const GemmParams& p, const GatherDesc& d, uint8_t* tile, uint32_t l,
                                            uint32_t line_major, uint32_t inner0, uint64_t batch_off) {
  uint8_t* line = tile + l * kLineBytes;
  // 16-byte chunk j of line l lands at chunk j ^ (l % 8); MN-major tf32 tiles swizzle 32-byte chunks by l % 4.
  const uint32_t sw = (p.tf32 && d.mn_major) ? ((l & 3) << 1) : (l & 7);
  const uint32_t epc = p.tf32 ? 4u : 8u;   // elements per 16-byte chunk
  GatherDesc src = d;
  src.base = (const uint8_t*)d.base + batch_off * (d.src_is_bf16 ? 2 : 4);
  const LineCtx ctx = make_line_ctx(src, p.geo, line_major);
  const bool convert = !p.tf32 && !src.src_is_bf16;   // f32 in memory, bf16 in the tile: two 16-byte loads per chunk
  uint4 lo[8], hi[8];
  uint32_t slow = 0;
#pragma unroll
  for (uint32_t chunk = 0; chunk < 8; ++chunk) {
    uint32_t run;
    const int64_t first = gather_run(src, p.geo, ctx, inner0 + chunk * epc, epc, run);
    lo[chunk] = make_uint4(0, 0, 0, 0);
    hi[chunk] = make_uint4(0, 0, 0, 0);
    if (run < epc) { slow |= 1u << chunk; continue; }
    if (first < 0) continue;
    const uint8_t* ptr = (const uint8_t*)src.base + first * (src.src_is_bf16 ? 2 : 4);
    if (((uintptr_t)ptr & 15) != 0 || (p.tf32 && src.src_is_bf16)) { slow |= 1u << chunk; continue; }
    lo[chunk] = *(const uint4*)ptr;
    if (convert) hi[chunk] = *(const uint4*)(ptr + 16);
  }
  // A patch operand that stands for a normalised-and-rectified map: in-bounds values become relu(scale * x + shift) in
  // bf16 (device.zig:1604-1612); padding stays exactly zero, which is why this cannot be done after a zero-filling copy.
  const bool affine = p.affine_scale != nullptr && d.source == kSrcPatch && !p.tf32 && src.src_is_bf16;
  uint32_t inbounds = 0;
  if (affine) {
#pragma unroll
    for (uint32_t chunk = 0; chunk < 8; ++chunk) {
      uint32_t run;
      if (gather_run(src, p.geo, ctx, inner0 + chunk * epc, epc, run) >= 0 && run == epc) inbounds |= 1u << chunk;
    }
  }
#pragma unroll
  for (uint32_t chunk = 0; chunk < 8; ++chunk) {
    uint4 out = lo[chunk];
    if (slow & (1u << chunk)) {
      float v[8];
      for (uint32_t e = 0; e < epc; ++e) {
        uint32_t run;
        const int64_t idx = gather_run(src, p.geo, ctx, inner0 + chunk * epc + e, 1, run);
        v[e] = load_as_f32(src, idx);
        if (affine && idx >= 0) {
          const uint32_t ci = (inner0 + chunk * epc + e) % p.geo.c;
          v[e] = bf16_to_f32((uint16_t)affine_relu_bf16x2(bf16_bits(v[e]), p.affine_scale[ci], p.affine_shift[ci]));
        }
      }
      if (p.tf32) out = make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3]));
      else out = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
    } else if (convert) {
      const uint4 a = lo[chunk], b2 = hi[chunk];
      out = make_uint4(pack_bf16x2(__uint_as_float(a.x), __uint_as_float(a.y)), pack_bf16x2(__uint_as_float(a.z), __uint_as_float(a.w)),
                       pack_bf16x2(__uint_as_float(b2.x), __uint_as_float(b2.y)), pack_bf16x2(__uint_as_float(b2.z), __uint_as_float(b2.w)));
    }
    if (affine && !(slow & (1u << chunk)) && (inbounds & (1u << chunk))) {
      const uint32_t ci = (inner0 + chunk * epc) % p.geo.c;   // a multiple of 8: the chunk is one aligned run of channels
      const uint4 sc = *(const uint4*)(p.affine_scale + ci), sh = *(const uint4*)(p.affine_shift + ci);
      out = make_uint4(affine_relu_bf16x2(out.x, sc.x, sh.x), affine_relu_bf16x2(out.y, sc.y, sh.y), affine_relu_bf16x2(out.z, sc.z, sh.z),
                       affine_relu_bf16x2(out.w, sc.w, sh.w));
    }
    sts128(smem_u32(line) + ((chunk ^ sw) << 4), out);
  }
}
// A line of the patch operand of a 3-channel 3x3 stride-1 layer over a bf16 map (the network's stem): the 27 values of a
// window are three runs of nine consecutive bf16 (the pixels x - 1 .. x + 1 of a row, three channels each), so the line
// is 27 two-byte loads issued together, packed and stored as four 16-byte chunks, the other four chunks zero.  (Through
// the general routine every chunk of such a line straddles taps and goes element by element through the index arithmetic.)
__device__ __forceinline__ bool stem_line_applies(const GemmParams& p, const GatherDesc& d) {
  const ConvGeo& g = p.geo;
  return d.source == kSrcPatch && d.src_is_bf16 && !p.tf32 && g.c == 3 && g.c_step == 3 && g.k == 3 && g.stride == 1 && g.dilation == 1 &&
         p.affine_scale == nullptr;
}
// The loads of one line: 27 values (v[27] = 0 pads the last pair).  One pointer per window row, constant offsets within
// it (the pixel pitch is 3), nine predicates; the position is split with the walk's precomputed divisors.
__device__ __forceinline__ void stem_line_load(const GemmParams& p, const GatherDesc& d, uint32_t position, uint16_t (&v)[28]) {
  const ConvGeo& g = p.geo;
  const uint32_t img = fast_div(position, p.walk.div_image), rem = position - img * p.walk.div_image.d;
  const uint32_t oy = fast_div(rem, p.walk.div_w), ox = rem - oy * p.walk.div_w.d;
  const int32_t y0 = (int32_t)oy - (int32_t)g.pad, x0 = (int32_t)ox - (int32_t)g.pad;
  const bool valid = position < d.lines_total;
  const int32_t row_pitch = (int32_t)(g.w * 3);
  const uint16_t* corner = (const uint16_t*)d.base + (int64_t)img * g.h * row_pitch + (int64_t)y0 * row_pitch + (int64_t)x0 * 3;   // may lie outside: read under predicates only
  bool col_in[3];
#pragma unroll
  for (uint32_t kx = 0; kx < 3; ++kx) col_in[kx] = x0 + (int32_t)kx >= 0 && x0 + (int32_t)kx < (int32_t)g.w;
#pragma unroll
  for (uint32_t ky = 0; ky < 3; ++ky) {
    const bool row_in = valid && y0 + (int32_t)ky >= 0 && y0 + (int32_t)ky < (int32_t)g.h;
    const uint16_t* row = corner + (int32_t)ky * row_pitch;
#pragma unroll
    for (uint32_t e = 0; e < 9; ++e) v[ky * 9 + e] = (row_in && col_in[e / 3]) ? row[e] : (uint16_t)0;
  }
  v[27] = 0;
}
// Two neighbouring positions of one output row share eight of their twelve window columns' values: one set of 36
// loads (three rows of four pixels) serves both lines.
__device__ __forceinline__ void stem_line_pair_load(const GemmParams& p, const GatherDesc& d, uint32_t position, uint32_t img, uint32_t oy,
                                                    uint32_t ox, uint16_t (&va)[28], uint16_t (&vb)[28]) {
  const ConvGeo& g = p.geo;
  const int32_t y0 = (int32_t)oy - (int32_t)g.pad, x0 = (int32_t)ox - (int32_t)g.pad;
  const bool valid_a = position < d.lines_total, valid_b = position + 1 < d.lines_total;
  const int32_t row_pitch = (int32_t)(g.w * 3);
  const uint16_t* corner = (const uint16_t*)d.base + (int64_t)img * g.h * row_pitch + (int64_t)y0 * row_pitch + (int64_t)x0 * 3;
  bool col_in[4];
#pragma unroll
  for (uint32_t kx = 0; kx < 4; ++kx) col_in[kx] = x0 + (int32_t)kx >= 0 && x0 + (int32_t)kx < (int32_t)g.w;
#pragma unroll
  for (uint32_t ky = 0; ky < 3; ++ky) {
    const bool row_in = valid_a && y0 + (int32_t)ky >= 0 && y0 + (int32_t)ky < (int32_t)g.h;
    const uint16_t* row = corner + (int32_t)ky * row_pitch;
    uint16_t w[12];
#pragma unroll
    for (uint32_t e = 0; e < 12; ++e) w[e] = (row_in && col_in[e / 3]) ? row[e] : (uint16_t)0;
#pragma unroll
    for (uint32_t e = 0; e < 9; ++e) {
      va[ky * 9 + e] = w[e];
      vb[ky * 9 + e] = valid_b ? w[e + 3] : (uint16_t)0;
    }
  }
  va[27] = 0;
  vb[27] = 0;
}
__device__ __forceinline__ void stem_line_store(uint8_t* tile, uint32_t l, const uint16_t (&v)[28]) {
  const uint32_t line = smem_u32(tile + l * kLineBytes), sw = l & 7;
#pragma unroll
  for (uint32_t chunk = 0; chunk < 8; ++chunk) {
    uint4 out = make_uint4(0u, 0u, 0u, 0u);
    if (chunk < 4) {
      uint32_t w[4];
#pragma unroll
      for (uint32_t j = 0; j < 4; ++j) {
        const uint32_t e = chunk * 8 + 2 * j;
        w[j] = (e < 28 ? (uint32_t)v[e] : 0u) | ((e + 1 < 28 ? (uint32_t)v[e + 1] : 0u) << 16);
      }
      out = make_uint4(w[0], w[1], w[2], w[3]);
    }
    sts128(line + ((chunk ^ sw) << 4), out);
  }
}

__device__ __forceinline__ void gather_tile(const GemmParams& p, const GatherDesc& d, uint8_t* tile, uint32_t lines_in_tile,
                                            uint32_t mn0, uint32_t k0, uint32_t batch, uint32_t tid) {
  const uint32_t epl = p.tf32 ? 32u : 64u;
  const uint64_t batch_off = (uint64_t)batch * d.batch_stride;
  // The stem: K-major (forward) its 27 values are the one K block of a position's line; MN-major (weight gradient) they
  // are the first 27 of the tile's 128 rows, one line per position of the K block, and the lines of rows 64.. are zero.
  if (batch_off == 0 && (d.mn_major ? mn0 == 0 : k0 == 0) && stem_line_applies(p, d)) {
    const uint32_t first = d.mn_major ? k0 : mn0, windows = d.mn_major ? min(lines_in_tile, epl) : lines_in_tile;
    if (windows <= kGatherThreads) {   // a line for every thread: sharing loads between neighbours would idle half of them
      if (tid < windows) {
        uint16_t v[28];
        stem_line_load(p, d, first + tid, v);
        stem_line_store(tile, tid, v);
      }
    } else
    for (uint32_t l = 2 * tid; l < windows; l += 2 * kGatherThreads) {   // lines l and l + 1
      const uint32_t position = first + l;
      const uint32_t img = fast_div(position, p.walk.div_image), rem = position - img * p.walk.div_image.d;
      const uint32_t oy = fast_div(rem, p.walk.div_w), ox = rem - oy * p.walk.div_w.d;
      uint16_t va[28], vb[28];
      if (ox + 1 < p.geo.out_w) {
        stem_line_pair_load(p, d, position, img, oy, ox, va, vb);
      } else {   // the second position starts the next row (or image): two windows of their own
        stem_line_load(p, d, position, va);
        stem_line_load(p, d, position + 1, vb);
      }
      stem_line_store(tile, l, va);
      if (l + 1 < windows) stem_line_store(tile, l + 1, vb);
    }
    for (uint32_t l = windows + tid; l < lines_in_tile; l += kGatherThreads) {
      const uint32_t line = smem_u32(tile + l * kLineBytes);
#pragma unroll
      for (uint32_t chunk = 0; chunk < 8; ++chunk) sts128(line + (chunk << 4), make_uint4(0u, 0u, 0u, 0u));
    }
    return;
  }
  for (uint32_t l = tid; l < lines_in_tile; l += kGatherThreads) {
    if (d.mn_major) {
      const uint32_t block = l / epl, kline = l - block * epl;
      gather_line(p, d, tile, l, k0 + kline, mn0 + block * epl, batch_off);
    } else {
      gather_line(p, d, tile, l, mn0 + l, k0, batch_off);
    }
  }
}

// ---- TMA issue ----------------------------------------------------------------------------------------
// One tile load, either on this CTA's own barrier or, for a CTA pair, on the pair leader's barrier.
template <bool kPair>
__device__ __forceinline__ void load_4d(uint8_t* dst, const CUtensorMap* tmap, uint64_t* bar, uint32_t pair_bar, int32_t x, int32_t y, int32_t z, int32_t w) {
  if constexpr (kPair) tma_pair_load_4d(smem_u32(dst), tmap, pair_bar, x, y, z, w);
  else tma_load_4d(dst, tmap, bar, x, y, z, w);
}

// ---- per-lane tile loads ----------------------------------------------------------------------------------
// The producer warp gives every TMA box of a stage to its own lane.  A lone thread runs dependent
// instructions at 5-10 cycles each, so what a lane does per K block must be short AND the same instruction
// stream in every lane, whatever operand its box belongs to: lanes that took different branches (a 4-D
// activation box beside a 3-D filter box, a switch over the operand kind) ran one after the other and the
// producer, not the copy engine, set the pace (~1000 cycles per K block for a convolution that needs 130-500).
// Hence: every tensor map has four dimensions (unused ones of extent 1), a box is four coordinates, and the
// walk along K is two nested counters with three precomputed coordinate steps:
//   A step  - neither counter wraps (next channel block, next 64 K values of a dense operand, next image rows)
//   B step  - the inner counter wraps (next tap column; next filter tap; next image)
//   C step  - both wrap (next tap row)
struct BoxLane {
  uint32_t active, smem_off;
  const CUtensorMap* tmap;
  int32_t x, y, z, w;
  uint32_t i0, n0, i1, n1;
  int32_t ax, ay, az, aw, bx, by, bz, bw, cx, cy, cz, cw;
  FastDiv per_image, grid_w;   // patch boxes: tile row -> (image, image row)
  uint32_t tap;                // column-patch stages: the tap (along y) whose B tile this box fills
};
constexpr uint32_t kNever = 0xFFFFFFFFu;

__device__ __forceinline__ uint32_t boxes_of(uint32_t kind, uint32_t lines, uint32_t epl) {
  if (kind == kGather) return 0;
  return (kind == kDenseMN || kind == kPatchMN) ? (epl == 64 ? lines >> 6 : lines >> 5) : 1u;   // epl is 64 or 32
}

// Once per kernel: which box this lane owns and how its coordinates step along K.
__device__ __forceinline__ void box_setup(const GemmParams& p, const TapWalk& walk, BoxLane& b, uint32_t lane, const CUtensorMap* tmap_a,
                                          const CUtensorMap* tmap_b, uint32_t b_lines, uint32_t& kind, uint32_t& index) {
  const int32_t epl = p.tf32 ? 32 : 64;
  const uint32_t nb_tap = boxes_of(p.b_kind, b_lines, epl);                   // B boxes of one tap
  const uint32_t na = boxes_of(p.a_kind, kBM, epl), nb = nb_tap * max(p.col_taps, 1u);
  b.active = lane < na + nb;
  const bool is_b = lane >= na;
  index = is_b ? lane - na : lane;
  kind = is_b ? p.b_kind : p.a_kind;
  b.tmap = is_b ? tmap_b : tmap_a;
  const uint32_t kmul = max(p.k_mul, 1u);
  const uint32_t a_bytes = p.a_stage_bytes ? p.a_stage_bytes : kATileBytes * kmul;
  const uint32_t b_tap = !p.col_taps ? 0u : (nb_tap <= 1 ? index : index / nb_tap);   // which tap's B tile this box fills
  b.tap = b_tap;
  if (p.col_taps && is_b) index -= b_tap * nb_tap;
  b.smem_off = (is_b ? a_bytes + b_tap * b_lines * kLineBytes : 0u) + index * epl * kLineBytes * kmul;
  b.n0 = b.n1 = kNever;
  b.i0 = b.i1 = 0;
  b.ax = b.ay = b.az = b.aw = b.bx = b.by = b.bz = b.bw = b.cx = b.cy = b.cz = b.cw = 0;
  b.x = b.y = b.z = b.w = 0;
  b.per_image = b.grid_w = FastDiv{1, 0};
  if (!b.active) return;
  if (kind == kPatchK) {
    b.per_image = walk.div_image;
    b.grid_w = walk.div_w;
  }
  if (p.col_taps && is_b) {
    // B of a column-patch plan: channel blocks innermost, then the next tap column; the tap along y is fixed.
    const int32_t cblocks = (int32_t)walk.cblocks, chan = cblocks * epl;
    b.n0 = walk.cblocks;
    const int32_t next_col = walk.tap_x * chan - (cblocks - 1) * epl;
    if (kind == kDenseK) { b.ax = epl; b.bx = next_col; }
    if (kind == kDenseMN) { b.ay = epl; b.by = next_col; }
    if (kind == kWeightK) { b.ax = epl; b.bx = -(cblocks - 1) * epl; b.bz = walk.tap_x; }
    return;
  }
  switch (kind) {
    case kDenseK: b.ax = epl; break;
    case kDenseMN: b.ay = epl * (int32_t)kmul; break;
    case kPatchK: {
      const int32_t cblocks = (int32_t)walk.cblocks;
      b.n0 = walk.cblocks; b.n1 = walk.n1;
      b.ax = epl;
      b.bx = -(cblocks - 1) * epl; b.by = walk.y_step;
      b.cx = b.bx; b.cy = -((int32_t)walk.n1 - 1) * walk.y_step; b.cz = walk.z_step;
      break;
    }
    case kWeightK: {
      const int32_t cblocks = (int32_t)walk.cblocks;
      b.n0 = walk.cblocks; b.n1 = walk.n1;
      b.ax = epl;
      b.bx = -(cblocks - 1) * epl; b.bz = walk.tap_x;
      b.cx = b.bx; b.cz = walk.tap_y - ((int32_t)walk.n1 - 1) * walk.tap_x;
      break;
    }
    case kPatchMN:
      if (p.box_n > 1) {
        b.aw = (int32_t)p.box_n;
      } else {
        const int32_t rows = (int32_t)(p.box_h * (p.patch_view ? 1u : p.geo.stride));
        b.n0 = p.geo.out_h / p.box_h;
        b.az = rows;
        b.bz = -((int32_t)b.n0 - 1) * rows; b.bw = 1;
      }
      break;
    default: break;
  }
}

// Once per tile: the box's coordinates and counters at K block work.kb_begin of a tile whose A rows start at m0
// and B lines at n0.
__device__ __forceinline__ void box_start(const GemmParams& p, const TapWalk& walk, BoxLane& b, uint32_t kind, uint32_t index, const Work& work,
                                          uint32_t m0, uint32_t n0, bool is_b) {
  if (!b.active) return;
  const uint32_t epl = p.tf32 ? 32u : 64u;
  const uint32_t mn0 = is_b ? n0 : m0;
  const uint32_t k0 = work.kb_begin * max(p.k_mul, 1u);   // in 64- (32-) wide K blocks
  b.i0 = b.i1 = 0;
  b.w = 0;
  if (p.col_taps) {   // column-patch plans never split K: every tile starts at the first tap column
    const int32_t tap = walk.tap0 + (int32_t)b.tap * walk.tap_y, chan = (int32_t)(walk.cblocks * epl);
    if (!is_b) {
      const uint32_t img = fast_div(mn0, b.per_image);
      const int32_t row0 = (int32_t)fast_div(mn0 - img * b.per_image.d, b.grid_w);
      const int32_t top = walk.z_step < 0 ? walk.z0 + ((int32_t)p.col_taps - 1) * walk.z_step : walk.z0;
      b.x = 0; b.y = walk.y0; b.z = row0 + top; b.w = (int32_t)img;
    } else if (kind == kDenseK) {
      b.x = tap * chan; b.y = (int32_t)mn0; b.z = 0;
    } else if (kind == kDenseMN) {
      b.x = (int32_t)(mn0 + index * epl); b.y = tap * chan; b.z = 0;
    } else {
      b.x = 0; b.y = (int32_t)mn0; b.z = tap;
    }
    return;
  }
  switch (kind) {
    case kDenseK:
      b.x = (int32_t)(k0 * epl); b.y = (int32_t)mn0;
      { uint32_t bi, bo; split_batch(p, work.batch, bi, bo); b.z = (int32_t)bi; b.w = (int32_t)bo; }
      break;
    case kDenseMN:
      b.x = (int32_t)(mn0 + index * epl); b.y = (int32_t)(k0 * epl);
      { uint32_t bi, bo; split_batch(p, work.batch, bi, bo); b.z = (int32_t)bi; b.w = (int32_t)bo; }
      break;
    case kPatchK: {
      uint32_t cb = 0, tx = 0, ty = 0;
      if (k0 != 0) {   // only a K split starts inside the tap walk
        const uint32_t tap = k0 / b.n0;
        cb = k0 - tap * b.n0;
        ty = tap / b.n1;
        tx = tap - ty * b.n1;
      }
      const uint32_t img = fast_div(mn0, b.per_image);
      const int32_t row0 = p.box_n > 1 ? 0 : (int32_t)(fast_div(mn0 - img * b.per_image.d, b.grid_w) * walk.row_scale);
      b.i0 = cb; b.i1 = tx;
      b.x = (int32_t)(cb * epl);
      b.y = walk.y0 + (int32_t)tx * walk.y_step;
      b.z = row0 + walk.z0 + (int32_t)ty * walk.z_step;
      b.w = (int32_t)img;
      break;
    }
    case kWeightK: {
      uint32_t cb = 0, tx = 0, ty = 0;
      if (k0 != 0) {
        const uint32_t tap = k0 / b.n0;
        cb = k0 - tap * b.n0;
        ty = tap / b.n1;
        tx = tap - ty * b.n1;
      }
      b.i0 = cb; b.i1 = tx;
      b.x = (int32_t)(cb * epl); b.y = (int32_t)mn0;
      b.z = walk.tap0 + (int32_t)tx * walk.tap_x + (int32_t)ty * walk.tap_y;
      break;
    }
    case kPatchMN: {
      // Rows (tap, channel) kk0 .. kk0 + epl of the weight gradient; rows past the last tap are never stored.
      const uint32_t taps = p.geo.k * p.geo.k, kk0 = mn0 + index * epl;
      const uint32_t tap = min(kk0 / p.geo.c, taps - 1);
      const uint32_t ky = tap / p.geo.k, kx = tap - ky * p.geo.k;
      const uint32_t per_image = p.geo.out_h * p.geo.out_w, p0 = k0 * epl;
      const uint32_t img = p0 / per_image;
      const uint32_t row = p.box_n > 1 ? 0u : (p0 - img * per_image) / p.geo.out_w;
      b.x = kk0 >= taps * p.geo.c ? 0 : (int32_t)(kk0 - tap * p.geo.c);
      b.y = (int32_t)(kx * p.geo.dilation) - (int32_t)p.geo.pad;
      b.z = (int32_t)(row * (p.patch_view ? 1u : p.geo.stride)) + (int32_t)(ky * p.geo.dilation) - (int32_t)p.geo.pad;
      b.w = (int32_t)img;
      b.i0 = p.box_n > 1 ? 0u : row / p.box_h;
      break;
    }
    default:
      break;
  }
}

// Steps the box to the next K block: the same dozen instructions in every lane.
__device__ __forceinline__ void box_step(BoxLane& b) {
  const uint32_t i0 = b.i0 + 1;
  const bool w0 = i0 == b.n0;
  const uint32_t i1 = b.i1 + (w0 ? 1u : 0u);
  const bool w1 = i1 == b.n1;
  b.i0 = w0 ? 0u : i0;
  b.i1 = w1 ? 0u : i1;
  b.x += w1 ? b.cx : (w0 ? b.bx : b.ax);
  b.y += w1 ? b.cy : (w0 ? b.by : b.ay);
  b.z += w1 ? b.cz : (w0 ? b.bz : b.az);
  b.w += w1 ? b.cw : (w0 ? b.bw : b.aw);
}

template <bool kPair>
__device__ __forceinline__ void box_issue(const BoxLane& b, uint8_t* stage_base, uint64_t* bar, uint32_t pair_bar) {
  load_4d<kPair>(stage_base + b.smem_off, b.tmap, bar, pair_bar, b.x, b.y, b.z, b.w);
}

// ---- epilogue -----------------------------------------------------------------------------------------
__device__ __forceinline__ float load_out(const void* base, uint32_t is_bf16, uint64_t idx) {
  return is_bf16 ? bf16_to_f32(((const uint16_t*)base)[idx]) : ((const float*)base)[idx];
}
__device__ __forceinline__ void store_out(void* base, uint32_t is_bf16, uint64_t idx, float v) {
  if (is_bf16) ((uint16_t*)base)[idx] = (uint16_t)bf16_bits(v);
  else ((float*)base)[idx] = v;
}

// Applies the epilogue to 32 accumulator columns of one row and stores them.  `bias_lane` is bias[col0 + lane]
// (one coalesced load per warp, fetched a chunk ahead by the caller); lanes trade it with shuffles, so every
// lane runs the arithmetic and only the memory accesses are guarded by `live`.
// Element offset of the start of product row `row` within one batch entry of C.
__device__ __forceinline__ uint64_t out_row_offset(const GemmParams& p, const RowMap& rm, uint32_t row) {
  if (!rm.enabled) return (uint64_t)row * p.ldc;
  const uint32_t img = fast_div(row, rm.per_image);
  const uint32_t rem = row - img * rm.per_image.d;
  const uint32_t i = fast_div(rem, rm.grid_w), j = rem - i * rm.grid_w.d;
  const uint64_t pixel = ((uint64_t)img * rm.h + i * rm.scale + rm.off_y) * rm.w + j * rm.scale + rm.off_x;
  return pixel * p.ldc;
}

__device__ __forceinline__ void epilogue_chunk(const GemmParams& p, const uint32_t (&acc)[32], uint32_t batch, uint32_t split,
                                               uint32_t row, uint32_t col0, float bias_lane, uint64_t row_off, uint32_t m_limit,
                                               bool as_partial) {
  if (col0 >= p.n) return;
  const bool live = row < m_limit;
  const uint32_t cols = min(32u, p.n - col0);
  if (as_partial) {
    if (!live) return;
    float* dst = p.partial + (((uint64_t)split * p.batch + batch) * p.m + row) * p.n + col0;
    if (cols == 32 && (p.n & 3) == 0) {
#pragma unroll
      for (uint32_t i = 0; i < 32; i += 4) *(uint4*)(dst + i) = make_uint4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
    } else {
      for (uint32_t i = 0; i < cols; ++i) dst[i] = __uint_as_float(acc[i]);
    }
    return;
  }
  const uint64_t cbase = c_batch_offset(p, batch);
  float v[32];
#pragma unroll
  for (uint32_t i = 0; i < 32; ++i) v[i] = __uint_as_float(acc[i]);
  const bool vec = p.vec_store && !p.transpose_out && cols == 32;
  if (vec) {
    const uint64_t off = cbase + row_off + col0;
    if (p.accumulate && live) {
      if (p.c_is_bf16) {
#pragma unroll
        for (uint32_t i = 0; i < 32; i += 8) {
          const uint4 q = *(const uint4*)((const uint16_t*)p.c + off + i);
          const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
          for (uint32_t j = 0; j < 4; ++j) {
            v[i + 2 * j] += __uint_as_float(w[j] << 16);
            v[i + 2 * j + 1] += __uint_as_float(w[j] & 0xFFFF0000u);
          }
        }
      } else {
#pragma unroll
        for (uint32_t i = 0; i < 32; i += 4) {
          const float4 q = *(const float4*)((const float*)p.c + off + i);
          v[i] += q.x; v[i + 1] += q.y; v[i + 2] += q.z; v[i + 3] += q.w;
        }
      }
    }
    if (p.bias) {
#pragma unroll
      for (uint32_t i = 0; i < 32; ++i) v[i] += __shfl_sync(0xFFFFFFFFu, bias_lane, i);
    }
    if (p.residual && live) {
      if (p.c_is_bf16) {
#pragma unroll
        for (uint32_t i = 0; i < 32; i += 8) {
          const uint4 q = *(const uint4*)((const uint16_t*)p.residual + off + i);
          const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
          for (uint32_t j = 0; j < 4; ++j) {
            v[i + 2 * j] += __uint_as_float(w[j] << 16);
            v[i + 2 * j + 1] += __uint_as_float(w[j] & 0xFFFF0000u);
          }
        }
      } else {
#pragma unroll
        for (uint32_t i = 0; i < 32; i += 4) {
          const float4 q = *(const float4*)((const float*)p.residual + off + i);
          v[i] += q.x; v[i + 1] += q.y; v[i + 2] += q.z; v[i + 3] += q.w;
        }
      }
    }
    if (p.relu) {
#pragma unroll
      for (uint32_t i = 0; i < 32; ++i) v[i] = fmaxf(v[i], 0.0f);
    }
    if (p.round_tf32) {
#pragma unroll
      for (uint32_t i = 0; i < 32; ++i) v[i] = round_tf32(v[i]);
    }
    if (!live) return;
    if (p.c_is_bf16) {
#pragma unroll
      for (uint32_t i = 0; i < 32; i += 8)
        *(uint4*)((uint16_t*)p.c + off + i) = make_uint4(pack_bf16x2(v[i], v[i + 1]), pack_bf16x2(v[i + 2], v[i + 3]),
                                                         pack_bf16x2(v[i + 4], v[i + 5]), pack_bf16x2(v[i + 6], v[i + 7]));
    } else {
#pragma unroll
      for (uint32_t i = 0; i < 32; i += 4) *(float4*)((float*)p.c + off + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
    }
    if (p.zero_fill > 1) {
      // the pixels (y + dy, x + dx), 0 <= dy, dx < s, beside this row's pixel belong to classes without taps: zero
      const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
      for (uint32_t dy = 0; dy < p.zero_fill; ++dy)
        for (uint32_t dx = dy == 0 ? 1u : 0u; dx < p.zero_fill; ++dx) {
          const uint64_t at = off + ((uint64_t)dy * p.rowmap.w + dx) * p.ldc;
          if (p.c_is_bf16) {
#pragma unroll
            for (uint32_t i = 0; i < 32; i += 8) *(uint4*)((uint16_t*)p.c + at + i) = zero;
          } else {
#pragma unroll
            for (uint32_t i = 0; i < 32; i += 4) *(uint4*)((float*)p.c + at + i) = zero;
          }
        }
    }
    return;
  }
  if (!live) return;
#pragma unroll
  for (uint32_t i = 0; i < 32; ++i) {
    if (i < cols) {
      const uint32_t col = col0 + i;
      const uint64_t idx = cbase + (p.transpose_out ? (uint64_t)col * p.ldc + row : row_off + col);
      float x = v[i];
      if (p.accumulate) x += load_out(p.c, p.c_is_bf16, idx);
      if (p.bias) x += p.bias[col];
      if (p.residual) x += load_out(p.residual, p.c_is_bf16, idx);
      if (p.relu) x = fmaxf(x, 0.0f);
      if (p.round_tf32) x = round_tf32(x);
      store_out(p.c, p.c_is_bf16, idx, x);
    }
  }
}

// The guarded path for a ragged chunk met on the TMA-store route.  It works on its own copy of the chunk: the
// guarded path indexes the values with a run-time index, which puts its array in local memory, and the
// caller's accumulator registers must not follow it there.
__device__ __noinline__ void epilogue_chunk_ragged(const GemmParams& p, const uint32_t* vals, uint32_t batch, uint32_t split, uint32_t row,
                                                   uint32_t col0, float bias_lane) {
  uint32_t copy[32];
#pragma unroll
  for (uint32_t i = 0; i < 32; ++i) copy[i] = vals[i];
  epilogue_chunk(p, copy, batch, split, row, col0, bias_lane, (uint64_t)row * p.ldc, p.m, p.splits > 1);
}
__device__ __forceinline__ void epilogue_chunk_copy(const GemmParams& p, const uint32_t (&acc)[32], uint32_t batch, uint32_t split, uint32_t row,
                                                    uint32_t col0, float bias_lane) {
  uint32_t spill[32];
#pragma unroll
  for (uint32_t i = 0; i < 32; ++i) spill[i] = acc[i];
  epilogue_chunk_ragged(p, spill, batch, split, row, col0, bias_lane);
}

// Full 32-column chunk of 32 rows through shared memory and one TMA store.  Straight from the accumulator
// layout a lane owns a row, so a warp-wide 16-byte store touches 32 different lines and fills half a sector
// of each; with all SMs storing at once that took as long again as the rest of the epilogue.  Here the warp
// parks the chunk in its 2 KB staging block as 32 rows of 64 bytes (64-byte swizzle: the eight lanes of a
// quarter-warp hit eight different 16-byte bank groups) and lane 0 hands it to the TMA unit, which writes whole
// rows and clips the box at the edges of C.  The block is reused as soon as the previous store has read it.
__device__ __forceinline__ void stage_and_store(const CUtensorMap* tmap_c, uint8_t* stage, const uint4 (&q)[4], uint32_t lane, int32_t x,
                                                int32_t y, int32_t z, int32_t w = -1) {   // w >= 0: a map with two batch levels
  if (lane == 0) bulk_wait_read_all();
  __syncwarp();
  const uint32_t sw = (lane >> 1) & 3;
  const uint32_t line = smem_u32(stage) + lane * 64;
#pragma unroll
  for (uint32_t j = 0; j < 4; ++j) sts128(line + ((j ^ sw) << 4), q[j]);
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0) {
    if (w >= 0) tma_store_4d(tmap_c, stage, x, y, z, w);
    else tma_store_3d(tmap_c, stage, x, y, z);
    bulk_commit_group();
  }
}

// ---- batch-norm statistics in the epilogue ------------------------------------------------------------------
// Per-channel sums of (v - shift) and (v - shift)^2 over the values the tile stores, the role of `statsTile`
// (src/gpu/device.zig:1505-1535).  In the accumulator layout a lane owns a ROW of the chunk, so the 32 column sums of
// the warp's 32 rows are formed by a transposing butterfly: in the step of distance d a lane keeps the half of its
// columns that its bit d selects and adds the partner's values for them; after five steps lane l holds column l's sum
// over the 32 rows (31 shuffles per quantity instead of 160).  The order of the additions is fixed by the layout.
__device__ __forceinline__ float column_sums(float (&t)[32], uint32_t lane) {
#pragma unroll
  for (uint32_t d = 16; d >= 1; d >>= 1) {
    const bool upper = (lane & d) != 0;
#pragma unroll
    for (uint32_t j = 0; j < d; ++j) {
      const float keep = upper ? t[j + d] : t[j], give = upper ? t[j] : t[j + d];
      t[j] = keep + __shfl_xor_sync(0xFFFFFFFFu, give, d);
    }
  }
  return t[0];
}

struct ChunkStats {
  float sum, squares;
};
// `v` = the values as stored (already rounded to the output type), `shift` = this chunk's 32 shift values in shared memory.
__device__ __forceinline__ ChunkStats chunk_stats(const float* v, const float* shift, bool live, uint32_t lane) {
  float t[32], q[32];
#pragma unroll
  for (uint32_t i = 0; i < 32; i += 4) {
    const float4 sh = *(const float4*)(shift + i);
    t[i] = live ? v[i] - sh.x : 0.0f; t[i + 1] = live ? v[i + 1] - sh.y : 0.0f;
    t[i + 2] = live ? v[i + 2] - sh.z : 0.0f; t[i + 3] = live ? v[i + 3] - sh.w : 0.0f;
  }
#pragma unroll
  for (uint32_t i = 0; i < 32; ++i) q[i] = t[i] * t[i];
  ChunkStats out;
  out.sum = column_sums(t, lane);
  out.squares = column_sums(q, lane);
  return out;
}

// The sums a batch-norm BACKWARD needs from the epilogue of the input-gradient product that feeds it, the role of
// `dxStatsTile` (src/gpu/device.zig:1537-1580): v = the stored gradient with respect to a normalised-and-rectified map
// that was never written, x = the raw map the norm ran on.  x_hat = (x - mean) * inv_std rebuilds the normalised value,
// gamma * x_hat + beta > 0 the ReLU mask; the masked gradient g and g * x_hat are summed per column.  The products and
// sums are rounded one by one (no fused multiply-add), like the reference's separate operations.
// This lane's 32 bf16 values of the batch-norm input (its row, the chunk's columns) for the masked gradient sums, fetched
// ahead of the accumulator they will be combined with: read inside the chunk routine, each chunk waited for them (a lane
// owns a row, so nothing else was in flight) and the pass took twice the plain input gradient.
__device__ __forceinline__ void dx_stats_fetch(const GemmParams& p, uint32_t batch, uint32_t row, uint32_t col0, uint4 (&raw)[4]) {
  const bool take = p.stats == 2 && row < p.m && col0 + 32 <= p.n;
  const uint16_t* src = (const uint16_t*)p.stat_x + c_batch_offset(p, batch) + (uint64_t)row * p.ldc + col0;
#pragma unroll
  for (uint32_t j = 0; j < 4; ++j) raw[j] = take ? *(const uint4*)(src + 8 * j) : make_uint4(0u, 0u, 0u, 0u);
}
__device__ __forceinline__ ChunkStats chunk_dx_stats(const float* v, const float* sstat, uint32_t slot, const uint4 (&xraw)[4], bool live, uint32_t lane) {
  const float *mean = sstat + 32 * slot, *inv_std = sstat + 384 + 32 * slot, *gamma = sstat + 512 + 32 * slot, *beta = sstat + 640 + 32 * slot;
  float t[32], q[32];
#pragma unroll
  for (uint32_t i = 0; i < 32; i += 4) {
    // four columns' parameters per 16-byte broadcast read (read one by one, the 128 shared-memory loads of a chunk
    // were the larger part of what this epilogue adds to the plain input gradient)
    const float4 m4 = *(const float4*)(mean + i), s4 = *(const float4*)(inv_std + i), g4 = *(const float4*)(gamma + i), b4 = *(const float4*)(beta + i);
    const float m[4] = {m4.x, m4.y, m4.z, m4.w}, is[4] = {s4.x, s4.y, s4.z, s4.w}, ga[4] = {g4.x, g4.y, g4.z, g4.w}, be[4] = {b4.x, b4.y, b4.z, b4.w};
    const uint4 raw = xraw[i / 8];
    const uint32_t w[2] = {(i & 4) ? raw.z : raw.x, (i & 4) ? raw.w : raw.y};
#pragma unroll
    for (uint32_t j = 0; j < 4; ++j) {
      const uint32_t c = i + j;
      const float x = __uint_as_float((j & 1) ? (w[j >> 1] & 0xFFFF0000u) : (w[j >> 1] << 16));
      const float xh = __fmul_rn(__fsub_rn(x, m[j]), is[j]);
      const bool on = live && __fadd_rn(__fmul_rn(ga[j], xh), be[j]) > 0.0f;
      t[c] = on ? v[c] : 0.0f;
      q[c] = on ? __fmul_rn(v[c], xh) : 0.0f;
    }
  }
  ChunkStats out;
  out.sum = column_sums(t, lane);
  out.squares = column_sums(q, lane);
  return out;
}

template <bool kStats>
__device__ __forceinline__ ChunkStats epilogue_chunk_tma_impl(const GemmParams& p, const CUtensorMap* tmap_c, const uint32_t (&acc)[32], uint8_t* stage,
                                                              const float* sbias, const float* sstat, uint32_t slot, const uint4 (&xraw)[4], uint32_t batch,
                                                              uint32_t split, uint32_t row, uint32_t col0, uint32_t lane) {
  ChunkStats stats = {0.0f, 0.0f};
  if (p.splits > 1) {
    // A K part's partial tile: the raw f32 accumulators, into the map of the partial buffer {n, m, split * batch}.
    // (Stored straight from the accumulator layout a lane owns a row and a warp-wide store half-fills 32 sectors:
    // with 29 parts of a weight gradient in flight those stores were most of the kernel.)
    const int32_t y = (int32_t)(row - lane), z = (int32_t)(split * p.batch + batch);
#pragma unroll
    for (uint32_t half = 0; half < 2; ++half) {
      uint4 q[4];
#pragma unroll
      for (uint32_t j = 0; j < 4; ++j) q[j] = make_uint4(acc[16 * half + 4 * j], acc[16 * half + 4 * j + 1], acc[16 * half + 4 * j + 2], acc[16 * half + 4 * j + 3]);
      stage_and_store(tmap_c, stage, q, lane, (int32_t)(col0 + 16 * half), y, z);
    }
    return stats;
  }
  const bool live = row < p.m;
  const uint64_t off = c_batch_offset(p, batch) + (uint64_t)row * p.ldc + col0;
  float v[32];
#pragma unroll
  for (uint32_t i = 0; i < 32; ++i) v[i] = __uint_as_float(acc[i]);
  if (p.accumulate && live) {
    if (p.c_is_bf16) {
#pragma unroll
      for (uint32_t i = 0; i < 32; i += 8) {
        const uint4 q = *(const uint4*)((const uint16_t*)p.c + off + i);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {
          v[i + 2 * j] += __uint_as_float(w[j] << 16);
          v[i + 2 * j + 1] += __uint_as_float(w[j] & 0xFFFF0000u);
        }
      }
    } else {
#pragma unroll
      for (uint32_t i = 0; i < 32; i += 4) {
        const float4 q = *(const float4*)((const float*)p.c + off + i);
        v[i] += q.x; v[i + 1] += q.y; v[i + 2] += q.z; v[i + 3] += q.w;
      }
    }
  }
  if (p.bias) {
#pragma unroll
    for (uint32_t i = 0; i < 32; i += 4) {
      const float4 b = *(const float4*)(sbias + i);   // same address in every lane: a broadcast read
      v[i] += b.x; v[i + 1] += b.y; v[i + 2] += b.z; v[i + 3] += b.w;
    }
  }
  if (p.residual && live) {
    if (p.c_is_bf16) {
#pragma unroll
      for (uint32_t i = 0; i < 32; i += 8) {
        const uint4 q = *(const uint4*)((const uint16_t*)p.residual + off + i);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {
          v[i + 2 * j] += __uint_as_float(w[j] << 16);
          v[i + 2 * j + 1] += __uint_as_float(w[j] & 0xFFFF0000u);
        }
      }
    } else {
#pragma unroll
      for (uint32_t i = 0; i < 32; i += 4) {
        const float4 q = *(const float4*)((const float*)p.residual + off + i);
        v[i] += q.x; v[i + 1] += q.y; v[i + 2] += q.z; v[i + 3] += q.w;
      }
    }
  }
  if (p.relu) {
#pragma unroll
    for (uint32_t i = 0; i < 32; ++i) v[i] = fmaxf(v[i], 0.0f);
  }
  if (p.round_tf32) {
#pragma unroll
    for (uint32_t i = 0; i < 32; ++i) v[i] = round_tf32(v[i]);
  }
  const int32_t y = (int32_t)(row - lane);
  int32_t bz = (int32_t)batch, bw = -1;
  if (p.batch_inner) { uint32_t bi, bo; split_batch(p, batch, bi, bo); bz = (int32_t)bi; bw = (int32_t)bo; }
  if (p.c_is_bf16) {
    uint4 q[4];
#pragma unroll
    for (uint32_t j = 0; j < 4; ++j)
      q[j] = make_uint4(pack_bf16x2(v[8 * j], v[8 * j + 1]), pack_bf16x2(v[8 * j + 2], v[8 * j + 3]), pack_bf16x2(v[8 * j + 4], v[8 * j + 5]),
                        pack_bf16x2(v[8 * j + 6], v[8 * j + 7]));
    if constexpr (kStats) {   // over the values as stored: the bf16-rounded ones (device.zig:1524)
      const uint32_t w[16] = {q[0].x, q[0].y, q[0].z, q[0].w, q[1].x, q[1].y, q[1].z, q[1].w, q[2].x, q[2].y, q[2].z, q[2].w, q[3].x, q[3].y, q[3].z, q[3].w};
#pragma unroll
      for (uint32_t j = 0; j < 16; ++j) {
        v[2 * j] = __uint_as_float(w[j] << 16);
        v[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
      }
      stats = p.stats == 2 ? chunk_dx_stats(v, sstat, slot, xraw, live, lane) : chunk_stats(v, sstat + 32 * slot, live, lane);
    }
    stage_and_store(tmap_c, stage, q, lane, (int32_t)col0, y, bz, bw);
  } else {
    if constexpr (kStats) stats = chunk_stats(v, sstat + 32 * slot, live, lane);   // the backward sums exist for bf16 maps only
#pragma unroll
    for (uint32_t half = 0; half < 2; ++half) {   // 16 f32 columns = 64 bytes per row and store
      uint4 q[4];
#pragma unroll
      for (uint32_t j = 0; j < 4; ++j)
        q[j] = make_uint4(__float_as_uint(v[16 * half + 4 * j]), __float_as_uint(v[16 * half + 4 * j + 1]), __float_as_uint(v[16 * half + 4 * j + 2]),
                          __float_as_uint(v[16 * half + 4 * j + 3]));
      stage_and_store(tmap_c, stage, q, lane, (int32_t)(col0 + 16 * half), y, bz, bw);
    }
  }
  return stats;
}

// The common chunk: bf16 result = max(acc + bias, floor), nothing read from global memory (p.tma_store == 2: no old C, no
// residual, no K split, no statistics).  Without a run-time branch per option the chunk is ~100 instructions instead
// of several hundred: bias values are always staged (zeros when there is no bias) and `floor` is 0 or -inf.
__device__ __forceinline__ void epilogue_chunk_fast(const CUtensorMap* tmap_c, const uint32_t (&acc)[32], uint8_t* stage, const float* sbias, float floor,
                                                    int32_t bz, int32_t bw, uint32_t row, uint32_t col0, uint32_t lane) {
  uint4 q[4];
#pragma unroll
  for (uint32_t j = 0; j < 4; ++j) {
    const float4 b0 = *(const float4*)(sbias + 8 * j), b1 = *(const float4*)(sbias + 8 * j + 4);   // same address in every lane: broadcast reads
    q[j] = make_uint4(pack_bf16x2(fmaxf(__uint_as_float(acc[8 * j]) + b0.x, floor), fmaxf(__uint_as_float(acc[8 * j + 1]) + b0.y, floor)),
                      pack_bf16x2(fmaxf(__uint_as_float(acc[8 * j + 2]) + b0.z, floor), fmaxf(__uint_as_float(acc[8 * j + 3]) + b0.w, floor)),
                      pack_bf16x2(fmaxf(__uint_as_float(acc[8 * j + 4]) + b1.x, floor), fmaxf(__uint_as_float(acc[8 * j + 5]) + b1.y, floor)),
                      pack_bf16x2(fmaxf(__uint_as_float(acc[8 * j + 6]) + b1.z, floor), fmaxf(__uint_as_float(acc[8 * j + 7]) + b1.w, floor)));
  }
  stage_and_store(tmap_c, stage, q, lane, (int32_t)col0, (int32_t)(row - lane), bz, bw);
}

__device__ __forceinline__ void epilogue_chunk_tma(const GemmParams& p, const CUtensorMap* tmap_c, const uint32_t (&acc)[32], uint8_t* stage,
                                                   const float* sbias, uint32_t batch, uint32_t split, uint32_t row, uint32_t col0, uint32_t lane) {
  const uint4 none[4] = {};
  epilogue_chunk_tma_impl<false>(p, tmap_c, acc, stage, sbias, nullptr, 0, none, batch, split, row, col0, lane);
}
// `sstat`, an epilogue warp's statistics block in shared memory (floats): [0, 128) the shift (or mean) values of its four
// column chunks, [128, 384) per chunk and lane the running (sum, sum of squares) of that lane's column over every row the
// warp has drained, and for the backward sums [384, 512) inv_std, [512, 640) gamma, [640, 768) beta.

// The bias values of every chunk this warp will drain from the next accumulator, fetched into the warp's own
// shared memory before it waits for that accumulator: chunk i's 32 values sit at sbias[32 * i].  (Fetched
// chunk by chunk from global memory, each load's latency stood between two chunks.)
__device__ __forceinline__ void stage_bias(const GemmParams& p, float* sbias, uint32_t ncols, uint32_t col_base, bool wide, uint32_t lane,
                                           uint32_t first, uint32_t step) {
  if (p.bias == nullptr && p.tma_store != 2) return;   // the branch-free chunk always adds: it gets zeros
  __syncwarp();
#pragma unroll
  for (uint32_t i = 0; i < 8; ++i) {
    const uint32_t c = first + i * step;
    if (c < ncols) {
      const uint32_t tc = wide ? ((c & 255) >> 7) * (ncols / 2) + (c >> 8) * 128 + (c & 127) : c;
      const uint32_t col = col_base + tc + lane;
      sbias[32 * i + lane] = (p.bias != nullptr && col < p.n) ? p.bias[col] : 0.0f;
    }
  }
  __syncwarp();
}

// Drains one accumulator of `ncols` columns: TMEM reads are double-buffered in registers (the next 32 columns
// are in flight while the current ones are processed) and the bias slice is fetched one chunk ahead.
// `wide` selects the column order of a two-half tile (see the pair kernel).  `release()` hands the accumulator
// back to the MMA issuer; it is called as soon as this warp's last TMEM read has landed in registers, before
// that chunk's arithmetic and stores: with short-K tiles (a convolution layer) the time from "accumulator
// full" to "accumulator free" is what paces the kernel.
template <bool kStats, class Release>
__device__ __forceinline__ void epilogue_tile(const GemmParams& p, uint32_t taddr, uint32_t ncols, uint32_t batch, uint32_t split,
                                              uint32_t row, uint32_t col_base, bool wide, uint32_t lane,
                                              uint32_t first, uint32_t step, const CUtensorMap* tmap_c, uint8_t* store_stage, const float* sbias,
                                              float* sstat, uint4 (&xraw)[4], Release release) {
  // a fused class product places its rows by its own map and ends at its own row count
  const RowMap& rowmap = p.n_classes ? p.cls[batch].rowmap : p.rowmap;
  const uint32_t m_limit = p.n_classes ? p.cls[batch].m : p.m;
  if (p.n_classes) batch = 0;   // the classes share one C: no batch stride
  if (first >= ncols) {
    release();
    return;
  }
  if (p.tma_store) {
    // Chunks that lie wholly inside C and rows that begin inside it go through the TMA store; a ragged last
    // chunk takes the guarded scalar path with its bias read back from the staged values.
    auto tile_col = [&](uint32_t c) { return wide ? ((c & 255) >> 7) * (ncols / 2) + (c >> 8) * 128 + (c & 127) : c; };
    if constexpr (kStats) {
      // One register buffer and the chunk routine inline: with two buffers, or with the routine out of line and its
      // accumulators handed over through local memory, the statistics pass took twice the plain pass.  `xraw` holds the
      // batch-norm input of the current chunk (mode 2; the caller fetched the first chunk's before it waited for the
      // accumulator), the next chunk's is requested before this chunk's accumulator values are waited for.
      uint32_t i = 0;
      for (uint32_t c = first; c < ncols; c += step, ++i) {
        uint32_t acc[32];
        tmem_ld_32x32(taddr + c, acc);
        uint4 xnext[4];
        dx_stats_fetch(p, batch, row, c + step < ncols ? col_base + tile_col(c + step) : p.n, xnext);
        tmem_ld_wait();
        if (c + step >= ncols) release();
        const uint32_t col0 = col_base + tile_col(c);
        if (col0 + 32 <= p.n && row - lane < p.m) {
          const ChunkStats s = epilogue_chunk_tma_impl<true>(p, tmap_c, acc, store_stage, sbias + 32 * i, sstat, i, xraw, batch, 0, row, col0, lane);
          float2* cell = (float2*)(sstat + 128) + i * 32 + lane;   // only this lane ever touches its cell
          float2 v = *cell;
          v.x += s.sum;
          v.y += s.squares;
          *cell = v;
        } else epilogue_chunk_copy(p, acc, batch, split, row, col0, p.bias ? sbias[32 * i + lane] : 0.0f);
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) xraw[j] = xnext[j];
      }
      return;
    }
    uint32_t acc_a[32], acc_b[32];
    tmem_ld_32x32(taddr + first, acc_a);
    uint32_t i = 0;
    const bool fast = p.tma_store == 2;
    const float floor = p.relu ? 0.0f : -INFINITY;
    int32_t bz = (int32_t)batch, bw = -1;
    if (p.batch_inner) { uint32_t bi, bo; split_batch(p, batch, bi, bo); bz = (int32_t)bi; bw = (int32_t)bo; }
    for (uint32_t c = first; c < ncols; c += 2 * step, i += 2) {
      const bool has_b = c + step < ncols;
      tmem_ld_wait();
      if (has_b) tmem_ld_32x32(taddr + c + step, acc_b);
      else release();
      {
        const uint32_t col0 = col_base + tile_col(c);
        if (col0 + 32 <= p.n && row - lane < p.m) {
          if (fast) epilogue_chunk_fast(tmap_c, acc_a, store_stage, sbias + 32 * i, floor, bz, bw, row, col0, lane);
          else epilogue_chunk_tma(p, tmap_c, acc_a, store_stage, sbias + 32 * i, batch, split, row, col0, lane);
        } else epilogue_chunk_copy(p, acc_a, batch, split, row, col0, p.bias ? sbias[32 * i + lane] : 0.0f);
      }
      if (has_b) {
        tmem_ld_wait();
        if (c + 2 * step < ncols) tmem_ld_32x32(taddr + c + 2 * step, acc_a);
        else release();
        const uint32_t col0 = col_base + tile_col(c + step);
        if (col0 + 32 <= p.n && row - lane < p.m) {
          if (fast) epilogue_chunk_fast(tmap_c, acc_b, store_stage, sbias + 32 * (i + 1), floor, bz, bw, row, col0, lane);
          else epilogue_chunk_tma(p, tmap_c, acc_b, store_stage, sbias + 32 * (i + 1), batch, split, row, col0, lane);
        } else epilogue_chunk_copy(p, acc_b, batch, split, row, col0, p.bias ? sbias[32 * (i + 1) + lane] : 0.0f);
      }
    }
    return;
  }
  auto tile_col = [&](uint32_t c) { return wide ? ((c & 255) >> 7) * (ncols / 2) + (c >> 8) * 128 + (c & 127) : c; };
  auto bias_at = [&](uint32_t c) {
    const uint32_t col = col_base + tile_col(c) + lane;
    return (p.bias != nullptr && c < ncols && col < p.n) ? p.bias[col] : 0.0f;
  };
  // This warp drains the 32-column chunks first, first + step, ...; two chunks are in flight (A and B registers).
  const uint64_t row_off = out_row_offset(p, rowmap, row);
  uint32_t acc_a[32], acc_b[32];
  float bias_next = bias_at(first);
  tmem_ld_32x32(taddr + first, acc_a);
  for (uint32_t c = first; c < ncols; c += 2 * step) {
    const bool has_b = c + step < ncols;
    tmem_ld_wait();
    if (has_b) tmem_ld_32x32(taddr + c + step, acc_b);
    else release();
    float bias_cur = bias_next;
    bias_next = bias_at(c + step);
    epilogue_chunk(p, acc_a, batch, split, row, col_base + tile_col(c), bias_cur, row_off, m_limit, p.splits > 1);
    if (has_b) {
      tmem_ld_wait();
      if (c + 2 * step < ncols) tmem_ld_32x32(taddr + c + 2 * step, acc_a);
      else release();
      bias_cur = bias_next;
      bias_next = bias_at(c + 2 * step);
      epilogue_chunk(p, acc_b, batch, split, row, col_base + tile_col(c + step), bias_cur, row_off, m_limit, p.splits > 1);
    }
  }
}

// Hands a warp's statistics over at the end of the kernel: added to sums[col] and sums[n + col] with atomics, or, for
// an ordered (reproducible) run, written to this warp's slot of the partial buffer that `stats_combine_kernel` adds
// up in CTA and warp order.
__device__ __noinline__ void flush_stats(const GemmParams& p, const float* sstat, uint32_t epi_warp, uint32_t lane, uint32_t first, uint32_t step) {
  for (uint32_t i = 0; i < 4; ++i) {
    const uint32_t col = first + i * step + lane;
    if (first + i * step >= p.bn || col >= p.n) continue;
    const float2 v = ((const float2*)(sstat + 128))[i * 32 + lane];
    if (p.stat_partial != nullptr) {
      float* dst = p.stat_partial + (((uint64_t)blockIdx.x * 8 + epi_warp) * 4 + i) * 64 + lane * 2;
      dst[0] = v.x;
      dst[1] = v.y;
    } else {
      atomicAdd(p.stat_sums + col, v.x);
      atomicAdd(p.stat_sums + p.n + col, v.y);
    }
  }
}

// ---- MMA issue loop -------------------------------------------------------------------------------------
// One thread feeds the tensor core, so the loop body must stay far below the 512 cycles a K block takes:
// descriptors are built once and advanced by adding byte offsets (>> 4) to their address field, and the
// barrier waits take the one-instruction path when the stage is already full.  (The first version
// rebuilt both descriptors for each of the four slices; its ~150 dependent instructions per K block
// capped the kernel at half the tensor rate.)
struct MmaSetup {
  uint32_t idesc;
  uint32_t a_step16, b_step16;      // descriptor increment per K slice (bytes >> 4)
  uint32_t stage16;                 // descriptor increment per pipeline stage
  uint64_t a_desc0, b_desc0;        // descriptors of stage 0, slice 0
};

__device__ __forceinline__ MmaSetup make_mma_setup(const GemmParams& p, uint32_t tile_rows, uint32_t instr_n, uint32_t tiles_addr, uint32_t stage_bytes,
                                                   uint32_t a_bytes) {
  const uint32_t epl = p.tf32 ? 32u : 64u;
  // K-major: the four K slices of a stage sit 32 bytes apart inside each line.  MN-major: a slice is 16
  // (bf16) or 8 (tf32) whole lines, and 64-/32-wide MN blocks follow each other every epl lines.
  const uint32_t slice_lines = p.tf32 ? 8u : 16u;
  const uint32_t kmul = max(p.k_mul, 1u);
  const uint32_t a_lbo = p.a_mn_major ? epl * kLineBytes * kmul : 16u, a_step = p.a_mn_major ? slice_lines * kLineBytes : 32u;
  const uint32_t b_lbo = p.b_mn_major ? epl * kLineBytes * kmul : 16u, b_step = p.b_mn_major ? slice_lines * kLineBytes : 32u;
  // MN-major tf32 tiles use the 32-byte-chunk swizzle whose atom is four lines (512 bytes).
  const uint32_t a_mode = (p.tf32 && p.a_mn_major) ? kSwizzle128Base32 : kSwizzle128, a_sbo = (p.tf32 && p.a_mn_major) ? 512u : 1024u;
  const uint32_t b_mode = (p.tf32 && p.b_mn_major) ? kSwizzle128Base32 : kSwizzle128, b_sbo = (p.tf32 && p.b_mn_major) ? 512u : 1024u;
  MmaSetup s;
  s.idesc = make_instr_desc(p.tf32 ? 2u : 1u, p.a_mn_major, p.b_mn_major, tile_rows, instr_n);
  s.a_step16 = a_step >> 4;
  s.b_step16 = b_step >> 4;
  s.stage16 = stage_bytes >> 4;
  s.a_desc0 = make_smem_desc(tiles_addr, a_lbo, a_sbo, a_mode);
  s.b_desc0 = make_smem_desc(tiles_addr + a_bytes, b_lbo, b_sbo, b_mode);
  return s;
}

// Issues the four K slices of one stage.
template <bool kPair, bool kTf32>
__device__ __forceinline__ void mma_stage(const MmaSetup& s, uint32_t tmem_d, uint32_t stage, uint32_t first_accumulate, uint32_t b_extra16 = 0,
                                          uint32_t a_extra16 = 0) {
  const uint64_t da = s.a_desc0 + (uint64_t)(stage * s.stage16 + a_extra16);
  const uint64_t db = s.b_desc0 + (uint64_t)(stage * s.stage16 + b_extra16);
  mma_issue<kPair, kTf32>(tmem_d, da, db, s.idesc, first_accumulate);
  mma_issue<kPair, kTf32>(tmem_d, da + s.a_step16, db + s.b_step16, s.idesc, 1u);
  mma_issue<kPair, kTf32>(tmem_d, da + 2 * s.a_step16, db + 2 * s.b_step16, s.idesc, 1u);
  mma_issue<kPair, kTf32>(tmem_d, da + 3 * s.a_step16, db + 3 * s.b_step16, s.idesc, 1u);
}
// The further K blocks of a stage that holds several (MN-major tiles: the next block is the next 64 / 32 lines).
template <bool kPair, bool kTf32>
__device__ __forceinline__ void mma_stage_more(const MmaSetup& s, uint32_t tmem_d, uint32_t stage, uint32_t kmul) {
  for (uint32_t t = 1; t < kmul; ++t) {
    const uint64_t da = s.a_desc0 + (uint64_t)(stage * s.stage16 + 4 * t * s.a_step16);
    const uint64_t db = s.b_desc0 + (uint64_t)(stage * s.stage16 + 4 * t * s.b_step16);
#pragma unroll
    for (uint32_t q = 0; q < 4; ++q) mma_issue<kPair, kTf32>(tmem_d, da + q * s.a_step16, db + q * s.b_step16, s.idesc, 1u);
  }
}

// ---- the kernel ---------------------------------------------------------------------------------------
// kStats = the instantiation whose epilogue also sums batch-norm statistics.  It is a kernel of its own because the mere
// presence of the (out-of-line) statistics call in the epilogue cost every other plan registers and spills: convolution
// layers ran 7-20 % slower with it compiled in, whether or not they asked for statistics.
template <bool kStats>
__global__ void __launch_bounds__(64 + 256 + kGatherThreads, 1)
gemm_sm100_kernel(const __grid_constant__ GemmParams p, const __grid_constant__ CUtensorMap tmap_a,
                  const __grid_constant__ CUtensorMap tmap_b, const __grid_constant__ CUtensorMap tmap_c) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // pointer arithmetic, no integer round trip: every pointer derived from it stays known as shared memory
  SmemHeader* hdr = (SmemHeader*)smem;
  uint8_t* tiles = smem + kHeaderBytes;
  const uint32_t kmul = max(p.k_mul, 1u);
  const uint32_t b_tile_bytes = p.bn * kLineBytes * kmul;
  const uint32_t a_bytes = p.a_stage_bytes ? p.a_stage_bytes : kATileBytes * kmul, b_tiles = max(p.col_taps, 1u);
  const uint32_t stage_bytes = a_bytes + b_tiles * b_tile_bytes;
  volatile uint32_t* abort_flag = &hdr->abort_flag;

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t epi_threads = 128 * p.epi_groups;
  const bool has_gather = p.a_kind == kGather || p.b_kind == kGather;   // the extra warps gather (else, with p.xform, they transform)
  const uint32_t total_work = p.tiles_m * p.tiles_n * p.batch * p.splits;
  const uint32_t tmem_cols = p.bn * 2 <= 32 ? 32u : (p.bn * 2 <= 64 ? 64u : (p.bn * 2 <= 128 ? 128u : (p.bn * 2 <= 256 ? 256u : 512u)));

  // The prologue is spread over three warps so that none of it queues behind another part: warp 2 initialises the
  // barriers, warp 1 allocates tensor memory, and the producer warp meanwhile works out which box each lane owns (a
  // first walk through ~150 cold instructions that used to follow the barrier set-up in the same thread).
  const uint32_t epl = p.tf32 ? 32u : 64u;
  BoxLane box;
  uint32_t box_kind = 0, box_index = 0;
  if (warp == 0) box_setup(p, p.walk, box, lane, &tmap_a, &tmap_b, p.bn, box_kind, box_index);
  if (threadIdx.x == 64) {
    const uint32_t full_count = 1 + (has_gather ? kGatherThreads / 32 : 0);
    for (uint32_t s = 0; s < p.stages; ++s) {
      mbar_init(&hdr->full[s], full_count);
      mbar_init(&hdr->empty[s], 1);
      mbar_init(&hdr->xfull[s], kGatherThreads / 32);
    }
    for (uint32_t b = 0; b < 2; ++b) {
      mbar_init(&hdr->acc_full[b], 1);
      mbar_init(&hdr->acc_empty[b], 4 * p.epi_groups);
    }
    hdr->abort_flag = 0;
    hdr->spin_limit = p.spin_limit ? p.spin_limit : kSpinLimit;
    fence_barrier_init();
    if (p.a_kind != kGather) prefetch_tmap(&tmap_a);
    if (p.b_kind != kGather) prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(&hdr->tmem_base, tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  // Everything above touched only this CTA's shared and tensor memory, so it may overlap the tail of the previous
  // kernel in the stream.  Each role goes on with what needs no global memory -- the producer's box set-up and first
  // tile decode, the issuer's descriptors -- and waits for the stream's earlier work only right before its first
  // global access: that set-up is a first walk through cold instructions (~2500 cycles) that a product of one or two
  // tiles cannot hide otherwise.  The MMA issuer touches shared and tensor memory only and never waits.
  grid_launch_dependents();
  const uint32_t tmem_base = hdr->tmem_base;

  if (warp == 0) {
    // ===== TMA producer: one lane per box =====
    const uint32_t tx_bytes = (p.a_kind != kGather ? (p.col_taps ? p.a_box_bytes : kATileBytes * kmul) : 0u) + (p.b_kind != kGather ? b_tiles * b_tile_bytes : 0u);
    const uint32_t n_boxes = boxes_of(p.a_kind, kBM, epl) + b_tiles * boxes_of(p.b_kind, p.bn, epl);
    if (lane < max(n_boxes, 1u)) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      uint32_t cur_class = 0xFFFFFFFFu;
      const bool box_is_b = lane >= boxes_of(p.a_kind, kBM, epl);
      uint32_t ready = 1;   // the first pass over the ring finds every stage free
      uint32_t issued = 0;
      bool waited = false;
      for (uint32_t w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
        const Work work = decode_work(p, w);
        if (work.empty) continue;
        if (p.n_classes && work.batch != cur_class) {   // a new class: its own K walk
          box_setup(p, p.cls[work.batch].walk, box, lane, &tmap_a, &tmap_b, p.bn, box_kind, box_index);
          cur_class = work.batch;
        }
        box_start(p, p.n_classes ? p.cls[work.batch].walk : p.walk, box, box_kind, box_index, work, work.m_tile * kBM, work.n_tile * p.bn, box_is_b);
        for (uint32_t kb = work.kb_begin; kb < work.kb_end; ++kb) {
          if (!(ok = mbar_wait_peeked(&hdr->empty[stage], phase ^ 1, ready, abort_flag, kStatusProducerTimeout))) break;
          uint32_t next_stage = stage + 1, next_phase = phase;
          if (next_stage == p.stages) { next_stage = 0; next_phase ^= 1; }
          const bool more = kb + 1 < work.kb_end || w + gridDim.x < total_work;
          ready = more ? mbar_try_wait(&hdr->empty[next_stage], next_phase ^ 1) : 0u;
          // Failure injection asked for by the host (a test of the time-out path): CTA 0 leaves out one K block's
          // copies, so the stage's "full" barrier never completes and the bounded waits downstream run out.
          const bool dropped = p.test_drop_kblock != 0 && blockIdx.x == 0 && issued == p.test_drop_kblock - 1;
          ++issued;
          if (lane == 0 && !dropped) mbar_arrive_expect_tx(&hdr->full[stage], tx_bytes);
          if (!waited) {   // the first copy is this warp's first global access; everything up to here ran beside the previous kernel
            grid_dependency_wait();
            waited = true;
          }
          if (box.active && !dropped) box_issue<false>(box, tiles + stage * stage_bytes, &hdr->full[stage], 0);
          box_step(box);
          stage = next_stage;
          phase = next_phase;
        }
      }
    }
  } else if (warp == 1) {
    // ===== MMA issuer =====
    // The issuing thread is chosen with elect.sync, not `lane == 0`: the compiler then keeps descriptors and
    // addresses in uniform registers, and one tcgen05.mma costs ~40-48 issue cycles instead of ~92.
    if (elect_one()) {
      const MmaSetup ms = make_mma_setup(p, kBM, p.bn, smem_u32(tiles), stage_bytes, a_bytes);
      uint64_t* const stage_ready = p.xform ? hdr->xfull : hdr->full;   // a transformed operand is ready one hand-off later
      uint32_t stage = 0, phase = 0, buf = 0, buf_phase = 0;
      bool ok = true;
      uint32_t ready = 0;   // the first stage is waited for in the ordinary way
      for (uint32_t w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
        const Work work = decode_work(p, w);
        if (work.empty) continue;
        if (!(ok = mbar_wait_fast(&hdr->acc_empty[buf], buf_phase ^ 1, abort_flag, kStatusMmaTimeout))) break;
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + buf * p.bn;
        for (uint32_t kb = work.kb_begin; kb < work.kb_end; ++kb) {
          if (!(ok = mbar_wait_peeked(&stage_ready[stage], phase, ready, abort_flag, kStatusMmaTimeout))) break;
          uint32_t next_stage = stage + 1, next_phase = phase;
          if (next_stage == p.stages) { next_stage = 0; next_phase ^= 1; }
          const bool more = kb + 1 < work.kb_end || w + gridDim.x < total_work;
          ready = more ? mbar_try_wait(&stage_ready[next_stage], next_phase) : 0u;
          tc_fence_after_sync();
          if (p.col_taps) {
            for (uint32_t t = 0; t < p.col_taps; ++t) {
              const uint32_t a16 = (uint32_t)(p.col_a_first16 + (int32_t)t * p.col_a_step16), b16 = t * (b_tile_bytes >> 4);
              if (p.tf32) mma_stage<false, true>(ms, tmem_d, stage, (kb > work.kb_begin) | (t > 0), b16, a16);
              else mma_stage<false, false>(ms, tmem_d, stage, (kb > work.kb_begin) | (t > 0), b16, a16);
            }
          } else if (p.tf32) {
            mma_stage<false, true>(ms, tmem_d, stage, kb > work.kb_begin);
            mma_stage_more<false, true>(ms, tmem_d, stage, kmul);
          } else {
            mma_stage<false, false>(ms, tmem_d, stage, kb > work.kb_begin);
            mma_stage_more<false, false>(ms, tmem_d, stage, kmul);
          }
          mma_commit(&hdr->empty[stage]);
          stage = next_stage;
          phase = next_phase;
        }
        if (!ok) break;
        mma_commit(&hdr->acc_full[buf]);
        if ((buf ^= 1) == 0) buf_phase ^= 1;
      }
    }
  } else if (warp < 2 + 4 * p.epi_groups) {
    // ===== epilogue =====
    grid_dependency_wait();   // bias, old C and residual are read and C is written from here on
    const uint32_t quarter = warp & 3;
    uint32_t buf = 0, buf_phase = 0;
    bool ok = true;
    const bool tma_out = p.tma_store != 0;
    uint8_t* epi_smem = tiles + p.stages * stage_bytes;
    uint8_t* store_stage = epi_smem + (warp - 2) * kStoreStageBytesPerWarp;
    float* sbias = (float*)(epi_smem + 8 * kStoreStageBytesPerWarp + (warp - 2) * kStoreBiasBytesPerWarp);
    if (tma_out && warp == 2 && lane == 0) prefetch_tmap(&tmap_c);
    uint32_t bias_tile = 0xFFFFFFFFu;   // the column tile whose bias values sit in shared memory
    // statistics plans have one column tile, so a warp's shift values are staged once (chunk i's 32 values at sstat[32 * i])
    // and its running sums sit behind them
    float* sstat = (float*)(epi_smem + kStoreSmemBytes + (warp - 2) * kStatBytesPerWarp);
    if constexpr (kStats) {
      for (uint32_t i = 0; i < 4; ++i) {
        const uint32_t col = ((warp - 2) >> 2) * 32 + i * 32 * p.epi_groups + lane;
        sstat[32 * i + lane] = col < p.n ? p.stat_shift[col] : 0.0f;
        ((float2*)(sstat + 128))[32 * i + lane] = make_float2(0.0f, 0.0f);
        if (p.stats == 2) {
          sstat[384 + 32 * i + lane] = col < p.n ? p.stat_inv_std[col] : 0.0f;
          sstat[512 + 32 * i + lane] = col < p.n ? p.stat_gamma[col] : 0.0f;
          sstat[640 + 32 * i + lane] = col < p.n ? p.stat_beta[col] : 0.0f;
        }
      }
      __syncwarp();
    }
    for (uint32_t w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
      const Work work = decode_work(p, w);
      if (work.empty) continue;
      if (tma_out && p.splits == 1 && bias_tile != work.n_tile) {
        stage_bias(p, sbias, p.bn, work.n_tile * p.bn, false, lane, ((warp - 2) >> 2) * 32, 32 * p.epi_groups);
        bias_tile = work.n_tile;
      }
      const uint32_t row = work.m_tile * kBM + quarter * 32 + lane;
      uint4 xraw[4] = {};
      if constexpr (kStats) dx_stats_fetch(p, work.batch, row, work.n_tile * p.bn + ((warp - 2) >> 2) * 32, xraw);
      ok = mbar_wait(&hdr->acc_full[buf], buf_phase, abort_flag, kStatusEpilogueTimeout);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + ((quarter * 32) << 16) + buf * p.bn;
      epilogue_tile<kStats>(p, taddr, p.bn, work.batch, work.split, row, work.n_tile * p.bn, false, lane,
                                               ((warp - 2) >> 2) * 32, 32 * p.epi_groups, &tmap_c, store_stage, sbias, sstat, xraw, [&] {
                                                 tc_fence_before_sync();
                                                 __syncwarp();
                                                 if (lane == 0) mbar_arrive(&hdr->acc_empty[buf]);
                                               });
      if ((buf ^= 1) == 0) buf_phase ^= 1;
    }
    if constexpr (kStats) if (ok) flush_stats(p, sstat, warp - 2, lane, ((warp - 2) >> 2) * 32, 32 * p.epi_groups);
    if (tma_out && lane == 0) bulk_wait_all();   // the staging block must outlive its last store
  } else if (has_gather) {
    // ===== gather warps =====
    grid_dependency_wait();
    const uint32_t tid = threadIdx.x - 64 - epi_threads;
    uint32_t stage = 0, phase = 0;
    bool ok = true;
    for (uint32_t w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
      const Work work = decode_work(p, w);
      if (work.empty) continue;
      for (uint32_t kb = work.kb_begin; kb < work.kb_end; ++kb) {
        ok = mbar_wait(&hdr->empty[stage], phase ^ 1, abort_flag, kStatusProducerTimeout);
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (!ok) break;
        uint8_t* a_tile = tiles + stage * stage_bytes;
        if (p.a_kind == kGather) gather_tile(p, p.ga, a_tile, kBM, work.m_tile * kBM, kb * epl, work.batch, tid);
        if (p.b_kind == kGather) gather_tile(p, p.gbsrc, a_tile + kATileBytes, p.bn, work.n_tile * p.bn, kb * epl, work.batch, tid);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&hdr->full[stage]);
        if (++stage == p.stages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (p.xform) {
    // ===== transform warps: relu(scale * x + shift) over each landed A tile, in place =====
    // The copy filled whatever lies outside the image with NaN; fma keeps it NaN and max(NaN, 0) is 0, so padding ends up
    // exactly zero and in-bounds values become what the normalised-and-rectified map would have held (src/gpu/device.zig:
    // 77-86, 1604-1612).  A line is 64 channels of one pixel (the channel block of this K block: blocks are innermost in
    // every K walk); its 16-byte chunk j sits at chunk j ^ (line % 8).
    // In a weight gradient the patch operand is MN-major: a line is still 64 channels of one pixel, but the channel block
    // belongs to the BOX (64 of the tile's (tap, channel) rows), not to the K block.
    grid_dependency_wait();
    const uint32_t tid = threadIdx.x - 64 - epi_threads;
    // The norm expanded into bf16 scale / shift tables behind the epilogue's shared memory, once per CTA (a plan with
    // p.xform always carries the four vectors).
    const uint32_t cpad = (p.geo.c + 7) & ~7u;
    uint16_t* table = (uint16_t*)(tiles + p.stages * stage_bytes + (p.tma_store ? kStoreSmemBytes : 0) + (p.stats ? 8 * kStatBytesPerWarp : 0));
    for (uint32_t ch = tid; ch < p.geo.c; ch += kGatherThreads) {
      const float sc = __fmul_rn(p.aff_gamma[ch], p.aff_inv_std[ch]);
      table[ch] = (uint16_t)bf16_bits(sc);
      table[cpad + ch] = (uint16_t)bf16_bits(__fsub_rn(p.aff_beta[ch], __fmul_rn(p.aff_mean[ch], sc)));
    }
    asm volatile("bar.sync 1, %0;" ::"r"(kGatherThreads) : "memory");   // the transform warps only
    const uint32_t table_scale = smem_u32(table), table_shift = smem_u32(table + cpad);
    auto norm_of = [&](uint32_t ch, uint4& sc, uint4& sh) {   // scale and shift of channels ch .. ch + 7
      sc = lds128(table_scale + 2 * ch);
      sh = lds128(table_shift + 2 * ch);
    };
    const uint32_t a_lines = (p.col_taps ? p.a_box_bytes : kATileBytes * kmul) / kLineBytes;
    const uint32_t cblocks = max(p.walk.cblocks, 1u), box_lines = 64 * kmul;
    uint32_t stage = 0, phase = 0;
    bool ok = true;
    for (uint32_t w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
      const Work work = decode_work(p, w);
      if (work.empty) continue;
      uint32_t cb = work.kb_begin % cblocks;
      const uint32_t row_base = (work.m_tile * kBM) % p.geo.c;   // MN-major: first channel of the tile's first box
      // Thread t owns physical chunk t % 8 of lines t / 8, t / 8 + 8, ...: line % 8 is the same for all of them, so the
      // thread's logical chunk (its eight channels within the block) is fixed and its scale / shift values are loaded
      // once per stage (per box of an MN-major operand), not once per chunk -- and before the wait for the stage, one
      // box ahead, so that their latency never stands between a landed tile and its rewrite.
      const uint32_t pc = tid & 7, l0 = tid >> 3, jch = pc ^ (l0 & 7);
      const uint32_t n_boxes = p.a_mn_major ? a_lines / box_lines : 1u, lines_per_box = p.a_mn_major ? box_lines : a_lines;
      auto channel0 = [&](uint32_t box) {
        if (!p.a_mn_major) return cb * 64;
        const uint32_t c0 = row_base + box * 64;
        return c0 >= p.geo.c ? c0 - p.geo.c : c0;
      };
      for (uint32_t kb = work.kb_begin; kb < work.kb_end; ++kb) {
        uint32_t c0 = channel0(0);
        uint4 sc, sh;
        norm_of(c0 + jch * 8, sc, sh);
        ok = mbar_wait(&hdr->full[stage], phase, abort_flag, kStatusProducerTimeout);
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (!ok) break;
        uint8_t* a_tile = tiles + stage * stage_bytes;
        for (uint32_t box = 0; box < n_boxes; ++box) {
          const uint4 sc_box = sc, sh_box = sh;
          if (box + 1 < n_boxes) {
            c0 = channel0(box + 1);
            norm_of(c0 + jch * 8, sc, sh);
          }
          const uint32_t base = smem_u32(a_tile + (box * lines_per_box + l0) * kLineBytes + pc * 16);
          const uint32_t rounds = (lines_per_box - l0 + 7) / 8;   // lines l0, l0 + 8, ... of this box
          auto rewrite = [&](const uint4& v) {
            return make_uint4(affine_relu_bf16x2(v.x, sc_box.x, sh_box.x), affine_relu_bf16x2(v.y, sc_box.y, sh_box.y),
                              affine_relu_bf16x2(v.z, sc_box.z, sh_box.z), affine_relu_bf16x2(v.w, sc_box.w, sh_box.w));
          };
          uint32_t r = 0;
          for (; r + 8 <= rounds; r += 8) {   // eight loads in flight, then eight rewrites
            uint4 v[8];
#pragma unroll
            for (uint32_t j = 0; j < 8; ++j) v[j] = lds128(base + (r + j) * 8 * kLineBytes);
#pragma unroll
            for (uint32_t j = 0; j < 8; ++j) sts128(base + (r + j) * 8 * kLineBytes, rewrite(v[j]));
          }
          for (; r < rounds; ++r) sts128(base + r * 8 * kLineBytes, rewrite(lds128(base + r * 8 * kLineBytes)));
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&hdr->xfull[stage]);
        if (++stage == p.stages) { stage = 0; phase ^= 1; }
        if (++cb == cblocks) cb = 0;
      }
    }
  }

  // ===== teardown =====
  __syncwarp();
  if (*abort_flag != 0) {
    // A wait gave up: let copies and MMAs already in flight land before shared and tensor memory go away.
    for (int i = 0; i < 64; ++i) __nanosleep(10000);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (threadIdx.x == 0 && hdr->abort_flag != 0 && p.status != nullptr) atomicCAS(p.status, 0u, hdr->abort_flag);
  if (warp == 1) tmem_dealloc(tmem_base, tmem_cols);
}

// ---- the CTA-pair kernel ------------------------------------------------------------------------------
// Two CTAs of a cluster (two neighbouring SMs) share one 256 x BN tile: CTA r owns rows r*128..r*128+127
// and columns r*BN/2.. of the B tile.  One tcgen05.mma.cta_group::2 (M = 256) issued by the leader reads
// A from each CTA's own shared memory and each half of B once, so every SM moves half as many B bytes
// through shared memory as in the single-CTA kernel -- the single-CTA 128 x 256 tile is bound by
// shared-memory bandwidth (operand reads plus TMA writes exceed 128 B/clk), this one is not.
// Both CTAs run their own TMA producer (own tiles only, bytes counted on the leader's "full" barrier)
// and their own epilogue (own 128 accumulator rows); only the leader issues MMAs and commits, once per
// CTA, to the "empty" and "accumulator full" barriers of both.
template <bool kStats>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(320, 1)
gemm_sm100_pair_kernel(const __grid_constant__ GemmParams p, const __grid_constant__ CUtensorMap tmap_a,
                       const __grid_constant__ CUtensorMap tmap_b, const __grid_constant__ CUtensorMap tmap_c) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // pointer arithmetic, no integer round trip: every pointer derived from it stays known as shared memory
  SmemHeader* hdr = (SmemHeader*)smem;
  uint8_t* tiles = smem + kHeaderBytes;
  // A tile wider than 256 columns is two 256-column halves accumulated side by side in TMEM by two MMAs per
  // K slice (one accumulator buffer instead of two, so the epilogue no longer overlaps the next tile's
  // mainloop, but a quarter fewer operand bytes cross the L2 fabric and shared memory per flop).  CTA r
  // supplies tile columns r*bn/2 .. (r+1)*bn/2; half h uses the h-th 128-line block of each CTA's share, so
  // accumulator column c of half h is tile column (c / 128) * (bn / 2) + h * 128 + c % 128.
  const uint32_t halves = p.bn > 256 ? 2u : 1u, bufs = halves == 2 ? 1u : 2u;
  const uint32_t b_lines = p.bn / 2;                 // this CTA's share of the B tile
  const uint32_t b_tile_bytes = b_lines * kLineBytes;
  const uint32_t a_bytes = p.a_stage_bytes ? p.a_stage_bytes : kATileBytes, b_tiles = max(p.col_taps, 1u);
  const uint32_t stage_bytes = a_bytes + b_tiles * b_tile_bytes;
  volatile uint32_t* abort_flag = &hdr->abort_flag;

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();
  const uint32_t pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const uint32_t total_work = p.tiles_m * p.tiles_n * p.batch * p.splits;
  const uint32_t tmem_cols = p.bn * 2 <= 32 ? 32u : (p.bn * 2 <= 64 ? 64u : (p.bn * 2 <= 128 ? 128u : (p.bn * 2 <= 256 ? 256u : 512u)));

  const uint32_t epl = p.tf32 ? 32u : 64u;
  BoxLane box;   // see the single-CTA kernel: the producer's box set-up runs beside the barrier and tensor-memory set-up
  uint32_t box_kind = 0, box_index = 0;
  if (warp == 0) box_setup(p, p.walk, box, lane, &tmap_a, &tmap_b, b_lines, box_kind, box_index);
  if (threadIdx.x == 64) {
    for (uint32_t s = 0; s < p.stages; ++s) {
      mbar_init(&hdr->full[s], 1);      // the leader's arrive.expect_tx covers both CTAs' bytes (used on the leader only)
      mbar_init(&hdr->empty[s], 1);     // one commit from the leader
    }
    for (uint32_t b = 0; b < 2; ++b) {
      mbar_init(&hdr->acc_full[b], 1);  // one commit from the leader
      mbar_init(&hdr->acc_empty[b], 8 * p.epi_groups); // every epilogue warp of both CTAs (used on the leader only)
    }
    hdr->abort_flag = 0;
    hdr->spin_limit = p.spin_limit ? p.spin_limit : kSpinLimit;
    fence_barrier_init();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    tmem_pair_alloc(&hdr->tmem_base, tmem_cols);
    tmem_pair_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();                   // the partner's barriers are initialised before anyone signals them
  tc_fence_after_sync();
  grid_launch_dependents();             // see the single-CTA kernel: each role waits before its first global access
  const uint32_t tmem_base = hdr->tmem_base;

  if (warp == 0) {
    // ===== TMA producer (both CTAs): one lane per box =====
    // The leader announces the bytes of both CTAs with a plain local arrive; the partner only issues its
    // copies against the leader's barrier.  (A cluster-scope release arrive from each producer made every K
    // block wait for the previous block's copies: 1 us per block.)  The partner cannot run a phase ahead:
    // its stage is freed by the leader's commit, which follows the end of the phase.
    const uint32_t tx_bytes = (p.col_taps ? p.a_box_bytes : kATileBytes) + b_tiles * b_tile_bytes;
    const uint32_t n_boxes = boxes_of(p.a_kind, kBM, epl) + b_tiles * boxes_of(p.b_kind, b_lines, epl);
    if (lane < n_boxes) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      uint32_t cur_class = 0xFFFFFFFFu;
      const bool box_is_b = lane >= boxes_of(p.a_kind, kBM, epl);
      uint32_t ready = 1;   // the first pass over the ring finds every stage free
      bool waited = false;
      for (uint32_t w = pair; ok && w < total_work; w += pairs) {
        const Work work = decode_work(p, w);
        if (work.empty) continue;
        if (p.n_classes && work.batch != cur_class) {   // a new class: its own K walk
          box_setup(p, p.cls[work.batch].walk, box, lane, &tmap_a, &tmap_b, b_lines, box_kind, box_index);
          cur_class = work.batch;
        }
        box_start(p, p.n_classes ? p.cls[work.batch].walk : p.walk, box, box_kind, box_index, work, work.m_tile * 2 * kBM + rank * kBM,
                  work.n_tile * p.bn + rank * b_lines, box_is_b);
        for (uint32_t kb = work.kb_begin; kb < work.kb_end; ++kb) {
          if (!(ok = mbar_wait_peeked(&hdr->empty[stage], phase ^ 1, ready, abort_flag, kStatusProducerTimeout))) break;
          uint32_t next_stage = stage + 1, next_phase = phase;
          if (next_stage == p.stages) { next_stage = 0; next_phase ^= 1; }
          const bool more = kb + 1 < work.kb_end || w + pairs < total_work;
          ready = more ? mbar_try_wait(&hdr->empty[next_stage], next_phase ^ 1) : 0u;
          if (lane == 0 && rank == 0) mbar_arrive_expect_tx(&hdr->full[stage], 2 * tx_bytes);
          if (!waited) {
            grid_dependency_wait();
            waited = true;
          }
          box_issue<true>(box, tiles + stage * stage_bytes, nullptr, map_to_cta(smem_u32(&hdr->full[stage]), 0));
          box_step(box);
          stage = next_stage;
          phase = next_phase;
        }
      }
    }
  } else if (warp == 1) {
    // ===== MMA issuer (leader CTA only) =====
    if (rank == 0 && elect_one()) {
      const MmaSetup ms = make_mma_setup(p, 2 * kBM, p.bn / halves, smem_u32(tiles), stage_bytes, a_bytes);
      const uint32_t acc_stride = p.bn / halves;
      uint32_t stage = 0, phase = 0, buf = 0, buf_phase = 0;
      bool ok = true;
      uint32_t ready = 0;
      for (uint32_t w = pair; ok && w < total_work; w += pairs) {
        const Work work = decode_work(p, w);
        if (work.empty) continue;
        if (!(ok = mbar_wait_fast(&hdr->acc_empty[buf], buf_phase ^ 1, abort_flag, kStatusMmaTimeout))) break;
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + buf * acc_stride;
        for (uint32_t kb = work.kb_begin; kb < work.kb_end; ++kb) {
          if (!(ok = mbar_wait_peeked(&hdr->full[stage], phase, ready, abort_flag, kStatusMmaTimeout))) break;
          uint32_t next_stage = stage + 1, next_phase = phase;
          if (next_stage == p.stages) { next_stage = 0; next_phase ^= 1; }
          const bool more = kb + 1 < work.kb_end || w + pairs < total_work;
          ready = more ? mbar_try_wait(&hdr->full[next_stage], next_phase) : 0u;
          tc_fence_after_sync();
          if (p.col_taps) {
            for (uint32_t t = 0; t < p.col_taps; ++t) {
              const uint32_t a16 = (uint32_t)(p.col_a_first16 + (int32_t)t * p.col_a_step16), b16 = t * (b_tile_bytes >> 4);
              if (p.tf32) mma_stage<true, true>(ms, tmem_d, stage, (kb > work.kb_begin) | (t > 0), b16, a16);
              else mma_stage<true, false>(ms, tmem_d, stage, (kb > work.kb_begin) | (t > 0), b16, a16);
            }
          } else if (p.tf32) mma_stage<true, true>(ms, tmem_d, stage, kb > work.kb_begin);
          else mma_stage<true, false>(ms, tmem_d, stage, kb > work.kb_begin);
          if (halves == 2) {   // second half: 128 B lines (16 KB) further on, 256 TMEM columns further on
            if (p.tf32) mma_stage<true, true>(ms, tmem_d + 256, stage, kb > work.kb_begin, (128 * kLineBytes) >> 4);
            else mma_stage<true, false>(ms, tmem_d + 256, stage, kb > work.kb_begin, (128 * kLineBytes) >> 4);
          }
          // One arrival on the "empty" barrier of both CTAs (mask 0b11): each producer may refill its stage.
          mma_pair_commit_both(&hdr->empty[stage], 3);
          stage = next_stage;
          phase = next_phase;
        }
        if (!ok) break;
        mma_pair_commit_both(&hdr->acc_full[buf], 3);
        if (++buf == bufs) { buf = 0; buf_phase ^= 1; }
      }
    }
  } else {
    // ===== epilogue (both CTAs, own 128 rows) =====
    grid_dependency_wait();
    const uint32_t quarter = warp & 3;
    uint32_t buf = 0, buf_phase = 0;
    bool ok = true;
    const bool tma_out = p.tma_store != 0;
    uint8_t* epi_smem = tiles + p.stages * stage_bytes;
    uint8_t* store_stage = epi_smem + (warp - 2) * kStoreStageBytesPerWarp;
    float* sbias = (float*)(epi_smem + 8 * kStoreStageBytesPerWarp + (warp - 2) * kStoreBiasBytesPerWarp);
    if (tma_out && warp == 2 && lane == 0) prefetch_tmap(&tmap_c);
    uint32_t bias_tile = 0xFFFFFFFFu;   // the column tile whose bias values sit in shared memory
    float* sstat = (float*)(epi_smem + kStoreSmemBytes + (warp - 2) * kStatBytesPerWarp);   // see the single-CTA kernel
    if constexpr (kStats) {
      for (uint32_t i = 0; i < 4; ++i) {
        const uint32_t col = ((warp - 2) >> 2) * 32 + i * 32 * p.epi_groups + lane;
        sstat[32 * i + lane] = col < p.n ? p.stat_shift[col] : 0.0f;
        ((float2*)(sstat + 128))[32 * i + lane] = make_float2(0.0f, 0.0f);
        if (p.stats == 2) {
          sstat[384 + 32 * i + lane] = col < p.n ? p.stat_inv_std[col] : 0.0f;
          sstat[512 + 32 * i + lane] = col < p.n ? p.stat_gamma[col] : 0.0f;
          sstat[640 + 32 * i + lane] = col < p.n ? p.stat_beta[col] : 0.0f;
        }
      }
      __syncwarp();
    }
    for (uint32_t w = pair; ok && w < total_work; w += pairs) {
      const Work work = decode_work(p, w);
      if (work.empty) continue;
      if (tma_out && p.splits == 1 && bias_tile != work.n_tile) {
        stage_bias(p, sbias, p.bn, work.n_tile * p.bn, halves == 2, lane, ((warp - 2) >> 2) * 32, 32 * p.epi_groups);
        bias_tile = work.n_tile;
      }
      const uint32_t row = work.m_tile * 2 * kBM + rank * kBM + quarter * 32 + lane;
      uint4 xraw[4] = {};
      if constexpr (kStats) dx_stats_fetch(p, work.batch, row, work.n_tile * p.bn + ((warp - 2) >> 2) * 32, xraw);   // statistics plans have no wide tiles
      ok = mbar_wait(&hdr->acc_full[buf], buf_phase, abort_flag, kStatusEpilogueTimeout);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + ((quarter * 32) << 16) + buf * (p.bn / halves);
      epilogue_tile<kStats>(p, taddr, p.bn, work.batch, work.split, row, work.n_tile * p.bn, halves == 2, lane,
                                               ((warp - 2) >> 2) * 32, 32 * p.epi_groups, &tmap_c, store_stage, sbias, sstat, xraw, [&] {
                                                 tc_fence_before_sync();
                                                 __syncwarp();
                                                 if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&hdr->acc_empty[buf]), 0));
                                               });
      if (++buf == bufs) { buf = 0; buf_phase ^= 1; }
    }
    if constexpr (kStats) if (ok) flush_stats(p, sstat, warp - 2, lane, ((warp - 2) >> 2) * 32, 32 * p.epi_groups);
    if (tma_out && lane == 0) bulk_wait_all();   // the staging block must outlive its last store
  }

  // ===== teardown =====
  __syncwarp();
  if (*abort_flag != 0) {
    for (int i = 0; i < 64; ++i) __nanosleep(10000);
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();                   // neither CTA leaves while the partner may still signal its barriers
  tc_fence_after_sync();
  if (threadIdx.x == 0 && hdr->abort_flag != 0 && p.status != nullptr) atomicCAS(p.status, 0u, hdr->abort_flag);
  if (warp == 1) tmem_pair_dealloc(tmem_base, tmem_cols);
}

// Ordered combine of split-K partials followed by the epilogue; one thread per output element.
// Takes the place of grad's `splitCombine` (src/gpu/device.zig:664-670), which only deterministic runs use.
__global__ void splitk_reduce_kernel(const GemmParams p) {
  grid_launch_dependents();
  grid_dependency_wait();
  const uint64_t per_batch = (uint64_t)p.m * p.n;
  const uint64_t total = per_batch * p.batch;
  for (uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (uint64_t)gridDim.x * blockDim.x) {
    const uint32_t batch = (uint32_t)(t / per_batch);
    const uint64_t r = t - (uint64_t)batch * per_batch;
    const uint32_t row = (uint32_t)(r / p.n), col = (uint32_t)(r - (uint64_t)row * p.n);
    float x = 0.0f;
    for (uint32_t s = 0; s < p.splits; ++s) x += p.partial[(uint64_t)s * total + t];
    const uint64_t idx = c_batch_offset(p, batch) + (p.transpose_out ? (uint64_t)col * p.ldc + row : (uint64_t)row * p.ldc + col);
    if (p.accumulate) x += load_out(p.c, p.c_is_bf16, idx);
    if (p.bias) x += p.bias[col];
    if (p.residual) x += load_out(p.residual, p.c_is_bf16, idx);
    if (p.relu) x = fmaxf(x, 0.0f);
    if (p.round_tf32) x = round_tf32(x);
    store_out(p.c, p.c_is_bf16, idx, x);
  }
}

// The same combine for MANY parts (a weight gradient splits its positions 14-29 ways, the stem's FMA kernel into one part
// per block): one thread per element would chain that many dependent-latency loads (29 parts: 9 us for a 576 x 64 matrix,
// a third of the layer's time).  Here a block is 32 consecutive elements x 8 part groups: warp g sums its eighth of
// the parts in part order, the eight group sums are added in group order.  The association is fixed by (parts, 8), so
// the result is reproducible; it is not the left-to-right sum of the kernel above.
constexpr uint32_t kReduceGroups = 8;
// Four columns per thread with 16-byte loads, the parts fetched four at a time and added in part order: the scalar kernel
// above spends two 64-bit divisions and one dependent 4-byte load per part on every element (13 us for the eight parts
// of a 2304 x 256 weight gradient, beside a product of 21 us).  For a row-major, 16-byte aligned result with n % 4 == 0.
__global__ void __launch_bounds__(256) splitk_reduce_vec4_kernel(const GemmParams p) {
  grid_launch_dependents();
  grid_dependency_wait();
  const uint32_t n4 = p.n >> 2;
  const uint64_t per_batch4 = (uint64_t)p.m * n4, total4 = per_batch4 * p.batch, total = total4 * 4;
  const float4* parts = (const float4*)p.partial;
  for (uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total4; t += (uint64_t)gridDim.x * blockDim.x) {
    float4 x = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    uint32_t sidx = 0;
    for (; sidx + 4 <= p.splits; sidx += 4) {
      const float4 v0 = parts[(uint64_t)sidx * total4 + t], v1 = parts[(uint64_t)(sidx + 1) * total4 + t], v2 = parts[(uint64_t)(sidx + 2) * total4 + t],
                   v3 = parts[(uint64_t)(sidx + 3) * total4 + t];
      x.x += v0.x; x.y += v0.y; x.z += v0.z; x.w += v0.w;
      x.x += v1.x; x.y += v1.y; x.z += v1.z; x.w += v1.w;
      x.x += v2.x; x.y += v2.y; x.z += v2.z; x.w += v2.w;
      x.x += v3.x; x.y += v3.y; x.z += v3.z; x.w += v3.w;
    }
    for (; sidx < p.splits; ++sidx) {
      const float4 v = parts[(uint64_t)sidx * total4 + t];
      x.x += v.x; x.y += v.y; x.z += v.z; x.w += v.w;
    }
    uint32_t batch = 0;
    uint64_t r = t;
    if (p.batch > 1) { batch = (uint32_t)(t / per_batch4); r = t - (uint64_t)batch * per_batch4; }
    const uint32_t row = (uint32_t)r / n4, col = ((uint32_t)r - row * n4) * 4;   // m * n / 4 < 2^32: checked by the launcher
    const uint64_t idx = (uint64_t)batch * p.stride_c + (uint64_t)row * p.ldc + col;
    float v[4] = {x.x, x.y, x.z, x.w};
    if (p.accumulate) {
      if (p.c_is_bf16) {
        const uint2 q = *(const uint2*)((const uint16_t*)p.c + idx);
        v[0] += __uint_as_float(q.x << 16); v[1] += __uint_as_float(q.x & 0xFFFF0000u); v[2] += __uint_as_float(q.y << 16); v[3] += __uint_as_float(q.y & 0xFFFF0000u);
      } else {
        const float4 q = *(const float4*)((const float*)p.c + idx);
        v[0] += q.x; v[1] += q.y; v[2] += q.z; v[3] += q.w;
      }
    }
    if (p.bias) {
      const float4 b = *(const float4*)(p.bias + col);
      v[0] += b.x; v[1] += b.y; v[2] += b.z; v[3] += b.w;
    }
    if (p.residual) {
      if (p.c_is_bf16) {
        const uint2 q = *(const uint2*)((const uint16_t*)p.residual + idx);
        v[0] += __uint_as_float(q.x << 16); v[1] += __uint_as_float(q.x & 0xFFFF0000u); v[2] += __uint_as_float(q.y << 16); v[3] += __uint_as_float(q.y & 0xFFFF0000u);
      } else {
        const float4 q = *(const float4*)((const float*)p.residual + idx);
        v[0] += q.x; v[1] += q.y; v[2] += q.z; v[3] += q.w;
      }
    }
#pragma unroll
    for (uint32_t i = 0; i < 4; ++i) {
      if (p.relu) v[i] = fmaxf(v[i], 0.0f);
      if (p.round_tf32) v[i] = round_tf32(v[i]);
    }
    if (p.c_is_bf16) *(uint2*)((uint16_t*)p.c + idx) = make_uint2(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]));
    else *(float4*)((float*)p.c + idx) = make_float4(v[0], v[1], v[2], v[3]);
  }
  (void)total;
}

// The grouped reduce (below) with four columns per lane: for the many-part weight gradients of narrow layers whose result
// allows 16-byte accesses (f32, row-major, n % 4 == 0, nothing but `accumulate` in the epilogue).
__global__ void __launch_bounds__(32 * kReduceGroups) splitk_reduce_grouped_vec4_kernel(const GemmParams p) {
  __shared__ float4 group_sum[kReduceGroups][32];
  grid_launch_dependents();
  grid_dependency_wait();
  const uint32_t n4 = p.n >> 2;
  const uint64_t total4 = (uint64_t)p.m * n4;   // one batch entry: checked by the launcher
  const float4* parts = (const float4*)p.partial;
  const uint32_t lane = threadIdx.x & 31, group = threadIdx.x >> 5;
  const uint32_t s_begin = (uint32_t)((uint64_t)p.splits * group / kReduceGroups), s_end = (uint32_t)((uint64_t)p.splits * (group + 1) / kReduceGroups);
  for (uint64_t t0 = (uint64_t)blockIdx.x * 32; t0 < total4; t0 += (uint64_t)gridDim.x * 32) {
    const uint64_t t = t0 + lane;
    float4 x = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (t < total4) {
      uint32_t sidx = s_begin;
      for (; sidx + 2 <= s_end; sidx += 2) {
        const float4 v0 = parts[(uint64_t)sidx * total4 + t], v1 = parts[(uint64_t)(sidx + 1) * total4 + t];
        x.x += v0.x; x.y += v0.y; x.z += v0.z; x.w += v0.w;
        x.x += v1.x; x.y += v1.y; x.z += v1.z; x.w += v1.w;
      }
      for (; sidx < s_end; ++sidx) {
        const float4 v = parts[(uint64_t)sidx * total4 + t];
        x.x += v.x; x.y += v.y; x.z += v.z; x.w += v.w;
      }
    }
    __syncthreads();
    group_sum[group][lane] = x;
    __syncthreads();
    if (group == 0 && t < total4) {
      x = group_sum[0][lane];
#pragma unroll
      for (uint32_t gi = 1; gi < kReduceGroups; ++gi) {
        const float4 v = group_sum[gi][lane];
        x.x += v.x; x.y += v.y; x.z += v.z; x.w += v.w;
      }
      const uint32_t row = (uint32_t)t / n4, col = ((uint32_t)t - row * n4) * 4;
      float4* dst = (float4*)((float*)p.c + (uint64_t)row * p.ldc + col);
      if (p.accumulate) {
        const float4 q = *dst;
        x.x += q.x; x.y += q.y; x.z += q.z; x.w += q.w;
      }
      *dst = x;
    }
  }
}

__global__ void __launch_bounds__(32 * kReduceGroups) splitk_reduce_grouped_kernel(const GemmParams p) {
  __shared__ float group_sum[kReduceGroups][32];
  grid_launch_dependents();
  grid_dependency_wait();
  const uint64_t per_batch = (uint64_t)p.m * p.n;
  const uint64_t total = per_batch * p.batch;
  const uint32_t lane = threadIdx.x & 31, group = threadIdx.x >> 5;
  const uint32_t s_begin = (uint32_t)((uint64_t)p.splits * group / kReduceGroups), s_end = (uint32_t)((uint64_t)p.splits * (group + 1) / kReduceGroups);
  for (uint64_t t0 = (uint64_t)blockIdx.x * 32; t0 < total; t0 += (uint64_t)gridDim.x * 32) {
    const uint64_t t = t0 + lane;
    float x = 0.0f;
    if (t < total) {
      const float* src = p.partial + t;
      uint32_t sidx = s_begin;
      for (; sidx + 4 <= s_end; sidx += 4) {
        const float v0 = src[(uint64_t)sidx * total], v1 = src[(uint64_t)(sidx + 1) * total], v2 = src[(uint64_t)(sidx + 2) * total],
                    v3 = src[(uint64_t)(sidx + 3) * total];
        x += v0; x += v1; x += v2; x += v3;
      }
      for (; sidx < s_end; ++sidx) x += src[(uint64_t)sidx * total];
    }
    __syncthreads();
    group_sum[group][lane] = x;
    __syncthreads();
    if (group == 0 && t < total) {
      x = group_sum[0][lane];
#pragma unroll
      for (uint32_t gi = 1; gi < kReduceGroups; ++gi) x += group_sum[gi][lane];
      const uint32_t batch = (uint32_t)(t / per_batch);
      const uint64_t r = t - (uint64_t)batch * per_batch;
      const uint32_t row = (uint32_t)(r / p.n), col = (uint32_t)(r - (uint64_t)row * p.n);
      const uint64_t idx = (uint64_t)batch * p.stride_c + (p.transpose_out ? (uint64_t)col * p.ldc + row : (uint64_t)row * p.ldc + col);
      if (p.accumulate) x += load_out(p.c, p.c_is_bf16, idx);
      if (p.bias) x += p.bias[col];
      if (p.residual) x += load_out(p.residual, p.c_is_bf16, idx);
      if (p.relu) x = fmaxf(x, 0.0f);
      if (p.round_tf32) x = round_tf32(x);
      store_out(p.c, p.c_is_bf16, idx, x);
    }
  }
}

// Ordered combine of the statistics partials (the role of `columnCombine`, src/gpu/device.zig:672-678).  One block per
// 32-column chunk; warp w adds, for its lane's column, the slots of the CTAs [w * per, (w + 1) * per) and of their four
// row quarters in ascending order, then warp 0 adds the warps' subtotals in warp order and the total into sums.  The
// order depends on the CTA count alone, never on timing.  (One thread per column walking every CTA took ~25 us for 148
// CTAs: its 592 dependent additions each waited for a load.)
constexpr uint32_t kCombineWarps = 16;
__global__ void __launch_bounds__(32 * kCombineWarps) stats_combine_kernel(const float* partial, float* sums, uint32_t ctas, uint32_t n, uint32_t epi_groups) {
  __shared__ float2 sub[kCombineWarps][32];
  grid_launch_dependents();
  grid_dependency_wait();
  const uint32_t chunk = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t group = chunk % epi_groups, slot = chunk / epi_groups;
  const uint32_t per = (ctas + kCombineWarps - 1) / kCombineWarps;
  const uint32_t begin = min(warp * per, ctas), end = min(begin + per, ctas);
  float s = 0.0f, q = 0.0f;
#pragma unroll 4
  for (uint32_t cta = begin; cta < end; ++cta) {
    float2 v[4];
#pragma unroll
    for (uint32_t quarter = 0; quarter < 4; ++quarter)
      v[quarter] = *(const float2*)(partial + (((uint64_t)cta * 8 + group * 4 + quarter) * 4 + slot) * 64 + lane * 2);
#pragma unroll
    for (uint32_t quarter = 0; quarter < 4; ++quarter) {
      s += v[quarter].x;
      q += v[quarter].y;
    }
  }
  sub[warp][lane] = make_float2(s, q);
  __syncthreads();
  const uint32_t col = chunk * 32 + lane;
  if (warp != 0 || col >= n) return;
  s = 0.0f;
  q = 0.0f;
#pragma unroll
  for (uint32_t w = 0; w < kCombineWarps; ++w) {
    s += sub[w][lane].x;
    q += sub[w][lane].y;
  }
  sums[col] += s;
  sums[n + col] += q;
}

}  // namespace

uint32_t gemm_grid_ctas(const GemmParams& p, int sm_count);

cudaError_t launch_stats_combine(const GemmParams& p, uint32_t ctas, cudaStream_t stream) {
  return launch_overlapped(stats_combine_kernel, dim3((p.n + 31) / 32), dim3(32 * kCombineWarps), 0, stream, (const float*)p.stat_partial, p.stat_sums,
                           ctas, p.n, p.epi_groups);
}

size_t gemm_smem_bytes(const GemmParams& p) {
  const size_t b_lines = p.cta_pair ? p.bn / 2 : p.bn;
  return 1024 /* alignment slack */ + kHeaderBytes +
         (size_t)p.stages * ((p.a_stage_bytes ? p.a_stage_bytes : kATileBytes * (p.k_mul ? p.k_mul : 1u)) +
                             (p.col_taps ? p.col_taps : 1u) * b_lines * kLineBytes * (p.k_mul ? p.k_mul : 1u)) +
         (p.tma_store ? kStoreSmemBytes : 0) + (p.stats ? 8 * kStatBytesPerWarp : 0) +
         (p.xform && p.aff_mean ? (size_t)4 * ((p.geo.c + 7) & ~7u) : 0);
}

// Co-resident 2-CTA clusters of the pair kernel for a given dynamic shared-memory size (cached per size).
static uint32_t max_resident_pairs(size_t smem_bytes, int sm_count) {
  static std::mutex guard;   // one handle per host thread, but this cache is shared by all of them
  std::lock_guard<std::mutex> lock(guard);
  static size_t cached_smem[8] = {};
  static int cached_pairs[8] = {};
  static int cached_device[8] = {-1, -1, -1, -1, -1, -1, -1, -1};
  int device = 0;
  cudaGetDevice(&device);
  for (int i = 0; i < 8; ++i)
    if (cached_device[i] == device && cached_smem[i] == smem_bytes) return (uint32_t)cached_pairs[i];
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)sm_count / 2 * 2, 1, 1);
  cfg.blockDim = dim3(320, 1, 1);
  cfg.dynamicSmemBytes = smem_bytes;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, gemm_sm100_pair_kernel<false>, &cfg) != cudaSuccess || clusters <= 0) {
    cudaGetLastError();
    clusters = sm_count / 2 > 8 ? sm_count / 2 - 8 : 1;   // conservative guess when the query is unavailable
  }
  if (getenv("GB_DEBUG")) fprintf(stderr, "[gradb200] resident 2-CTA clusters at %zu B smem: %d (SMs %d)\n", smem_bytes, clusters, sm_count);
  static int next = 0;
  const int slot = next++ % 8;
  cached_device[slot] = device;
  cached_smem[slot] = smem_bytes;
  cached_pairs[slot] = clusters;
  return (uint32_t)clusters;
}

cudaError_t gemm_sm100_configure() {
  cudaError_t e = cudaFuncSetAttribute(gemm_sm100_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_sm100_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_sm100_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_sm100_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
  return e;
}

// CTAs the launch below uses (what the statistics partial buffer is sized by).
uint32_t gemm_grid_ctas(const GemmParams& p, int sm_count) {
  const uint32_t total_work = p.tiles_m * p.tiles_n * p.batch * p.splits;
  if (p.cta_pair) return 2 * std::min<uint32_t>(total_work, max_resident_pairs(gemm_smem_bytes(p), sm_count));
  return total_work < (uint32_t)sm_count ? total_work : (uint32_t)sm_count;
}

cudaError_t launch_gemm_sm100(const GemmParams& p, const CUtensorMap& tmap_a, const CUtensorMap& tmap_b, const CUtensorMap& tmap_c, int sm_count,
                              cudaStream_t stream) {
  const uint32_t total_work = p.tiles_m * p.tiles_n * p.batch * p.splits;
  if (total_work == 0) return cudaSuccess;
  if (p.cta_pair) {
    // tiles_m counts 256-row tiles here; one cluster of two CTAs per SM pair, persistent over the tiles.
    // A persistent grid must not exceed what the device can keep resident at once: the number of
    // co-resident 2-CTA clusters can be below sm_count / 2 (SMs are paired within a GPC), and a cluster
    // left waiting would run its whole share of tiles after the others have finished.
    const uint32_t pairs = std::min<uint32_t>(total_work, max_resident_pairs(gemm_smem_bytes(p), sm_count));
    return launch_overlapped(p.stats ? gemm_sm100_pair_kernel<true> : gemm_sm100_pair_kernel<false>, dim3(2 * pairs), dim3(64 + 128 * p.epi_groups),
                             gemm_smem_bytes(p), stream, p, tmap_a, tmap_b, tmap_c);
  }
  const bool gather = p.a_kind == kGather || p.b_kind == kGather;
  const uint32_t grid = total_work < (uint32_t)sm_count ? total_work : (uint32_t)sm_count;
  auto kernel = p.stats ? gemm_sm100_kernel<true> : gemm_sm100_kernel<false>;
  // the extra warps gather operands TMA cannot fetch, or rewrite landed tiles of a transformed operand
  return launch_overlapped(kernel, dim3(grid), dim3(64 + 128 * p.epi_groups + ((gather || p.xform) ? kGatherThreads : 0)), gemm_smem_bytes(p), stream, p, tmap_a,
                           tmap_b, tmap_c);
}

cudaError_t launch_splitk_reduce(const GemmParams& p, cudaStream_t stream) {
  const uint64_t total = (uint64_t)p.m * p.n * p.batch;
  if (total == 0) return cudaSuccess;
  if (p.splits >= 3 * kReduceGroups) {
    if (p.vec_store && !p.transpose_out && !p.c_is_bf16 && p.batch == 1 && (p.n & 3) == 0 && (p.ldc & 3) == 0 && !p.bias && !p.residual && !p.relu &&
        !p.round_tf32 && total / 4 < 0xFFFFFFFFull && total / 4 >= 148 * 32 && ((uintptr_t)p.partial & 15) == 0) {   // enough groups of four to fill the machine
      const uint64_t total4 = total / 4;
      const uint32_t blocks4 = (uint32_t)((total4 + 31) / 32 < 148 * 16 ? (total4 + 31) / 32 : 148 * 16);
      return launch_overlapped(splitk_reduce_grouped_vec4_kernel, dim3(blocks4), dim3(32 * kReduceGroups), 0, stream, p);
    }
    const uint32_t blocks = (uint32_t)((total + 31) / 32 < 148 * 32 ? (total + 31) / 32 : 148 * 32);
    return launch_overlapped(splitk_reduce_grouped_kernel, dim3(blocks), dim3(32 * kReduceGroups), 0, stream, p);
  }
  // 16-byte path: row-major result, every pointer and pitch 16-byte aligned (vec_store), whole groups of four columns
  if (p.splits >= 1 && p.batch_inner == 0 && p.vec_store && !p.transpose_out && (p.n & 3) == 0 && (p.ldc & 3) == 0 && (p.stride_c & 3) == 0 &&
      (uint64_t)p.m * p.n / 4 < 0xFFFFFFFFull && ((uintptr_t)p.partial & 15) == 0) {
    const uint64_t total4 = total / 4;
    const uint32_t blocks4 = (uint32_t)((total4 + 255) / 256 < 148 * 8 ? (total4 + 255) / 256 : 148 * 8);
    return launch_overlapped(splitk_reduce_vec4_kernel, dim3(blocks4), dim3(256), 0, stream, p);
  }
  const uint32_t blocks = (uint32_t)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  return launch_overlapped(splitk_reduce_kernel, dim3(blocks), dim3(256), 0, stream, p);
}

}  // namespace gb
