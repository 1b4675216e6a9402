// Thin inline-PTX wrappers for the sm_100a features the contraction kernels use: mbarriers with
// bounded waits, TMA tile loads, tensor memory (TMEM) management, tcgen05.mma issue/commit and
// the tcgen05.ld epilogue path.  Everything here is a direct spelling of one PTX instruction.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace gb {

// Device status codes written to the handle's status word when a bounded wait gives up.
enum : uint32_t {
  kStatusOk = 0,
  kStatusProducerTimeout = 1,   // TMA / gather producer never saw a free stage
  kStatusMmaTimeout = 2,        // MMA issuer never saw a full stage or a drained accumulator
  kStatusEpilogueTimeout = 3,   // epilogue never saw a finished accumulator
  kStatusDrainTimeout = 4,
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint32_t elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "elect.sync _|p, 0xFFFFFFFF;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(pred));
  return pred;
}

// ---- mbarrier -----------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done;
}

// Every wait in these kernels is bounded: after a limit of failed polls (kSpinLimit, about a second at worst)
// the waiter raises the shared abort flag, records a status code and returns false; every other waiter
// sees the flag within one poll and leaves its loop too, so a broken pipeline ends the kernel with an
// error status instead of hanging the device.  The limit sits in shared memory in the word after the abort
// flag (the kernels set it up with the flag), so a caller may shorten it per launch.
constexpr uint32_t kSpinLimit = 1u << 22;

static __device__ __noinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, uint32_t code) {
  const uint32_t limit = abort_flag[1];
  for (uint32_t spin = 0; spin < limit; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag != 0) return false;
    if (spin > 64) __nanosleep(spin > 4096 ? 256 : 32);
  }
  atomicCAS((uint32_t*)abort_flag, 0u, code);
  return false;
}
// Hot-loop flavour: the common case (the phase has already completed) costs one try_wait.
__device__ __forceinline__ bool mbar_wait_fast(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, uint32_t code) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, abort_flag, code);
}

// Pipelined flavour.  A poll whose result feeds a branch costs the issuing thread 100-250 cycles (the round
// trip to the barrier), more than the 40-50 cycles of a tcgen05.mma issue or the ~95 of a 16 KB TMA box.  The
// per-stage loops therefore poll the NEXT stage's barrier before they issue the current stage's work and pass
// the answer in here one iteration later; only a poll that came back "not yet" falls into the spinning wait.
__device__ __forceinline__ bool mbar_wait_peeked(uint64_t* bar, uint32_t parity, uint32_t peeked, volatile uint32_t* abort_flag, uint32_t code) {
  if (peeked) return true;
  return mbar_wait_slow(bar, parity, abort_flag, code);
}

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, uint32_t code) {
  const uint32_t limit = abort_flag[1];
  for (uint32_t spin = 0; spin < limit; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag != 0) return false;
    if (spin > 64) __nanosleep(spin > 4096 ? 256 : 32);
  }
  atomicCAS((uint32_t*)abort_flag, 0u, code);
  return false;
}

// Two IEEE fused multiply-adds in one instruction (sm_100: fma.rn.f32x2 on register pairs): the same bits as two scalar
// FMAs at half the issue slots, which is what bounds the CUDA-core kernels (64 FMAs against four or five 16-byte shared-memory
// reads per K value and thread).
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}

// ---- programmatic dependent launch ---------------------------------------------------------------
// A kernel launched with the programmatic-serialization attribute may start while its predecessor in the stream
// is still running; `grid_dependency_wait` returns once every predecessor has completed and its memory is
// visible, `grid_launch_dependents` lets the successor start being scheduled.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- proxies and fences -------------------------------------------------------------------------
// 16-byte accesses in the shared state space proper.  Through a generic pointer (the tiles are reached by pointer
// arithmetic on the dynamic shared-memory base, so the compiler cannot tell the space) the in-place rewrite of a landed
// tile ran at two thirds of this speed.  Volatile, without a memory clobber: the statements keep their order among
// themselves and relative to the barrier waits, arrivals and fences (volatile too), which is all their callers need,
// and a caller that wants several loads in flight issues them back to back before the first use.
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, const uint4& v) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w));
}

// Generic-proxy shared-memory writes (st.shared) become visible to the async proxy (TMA, tcgen05.mma).
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---- TMA tile loads (no cluster broadcast: each CTA fetches its own tiles) ------------------------
__device__ __forceinline__ void prefetch_tmap(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)tmap) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const void* tmap, uint64_t* bar, int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"((uint64_t)tmap), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const void* tmap, uint64_t* bar, int32_t x, int32_t y, int32_t z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"((uint64_t)tmap), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
// ---- TMA tile stores (shared -> global), tracked by the issuing thread's bulk async-groups ---------
__device__ __forceinline__ void tma_store_3d(const void* tmap, const void* src, int32_t x, int32_t y, int32_t z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"((uint64_t)tmap), "r"(smem_u32(src)), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void tma_store_4d(const void* tmap, const void* src, int32_t x, int32_t y, int32_t z, int32_t w) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               ::"l"((uint64_t)tmap), "r"(smem_u32(src)), "r"(x), "r"(y), "r"(z), "r"(w)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Returns once every committed store of this thread has finished READING its shared-memory source.
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// Returns once every committed store of this thread has completed.
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void tma_load_4d(void* dst, const void* tmap, uint64_t* bar, int32_t x, int32_t y, int32_t z, int32_t w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)), "l"((uint64_t)tmap), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}

// The same loads for a CTA pair (cta_group::2): `dst` is this CTA's own shared memory, `bar_addr` a
// shared::cluster address that may name the partner CTA's mbarrier (the pair's leader collects the bytes
// of both CTAs on one barrier).  Each CTA still fetches only its own tiles.
__device__ __forceinline__ void tma_pair_load_3d(uint32_t dst, const void* tmap, uint32_t bar_addr, int32_t x, int32_t y, int32_t z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"((uint64_t)tmap), "r"(bar_addr), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_pair_load_4d(uint32_t dst, const void* tmap, uint32_t bar_addr, int32_t x, int32_t y, int32_t z, int32_t w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"((uint64_t)tmap), "r"(bar_addr), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}

// ---- thread-block clusters ------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_addr) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx_cluster(uint32_t bar_addr, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.release.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(bar_addr), "r"(bytes) : "memory");
}

// ---- tensor memory --------------------------------------------------------------------------------
// Allocation is warp-wide (.sync.aligned): one whole warp calls it, the base address lands in smem.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(columns) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}

// CTA-pair flavours: both CTAs of the pair call these with the same arguments from the same warp index.
__device__ __forceinline__ void tmem_pair_alloc(uint32_t* smem_result, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(columns) : "memory");
}
__device__ __forceinline__ void tmem_pair_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_pair_dealloc(uint32_t base, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}

// ---- tcgen05.mma ----------------------------------------------------------------------------------
// Shared-memory matrix descriptor for an operand tile made of 128-byte lines.  Field layout (PTX ISA,
// tcgen05 shared memory descriptor): [0,14) start address >> 4, [16,30) leading byte offset >> 4,
// [32,46) stride byte offset >> 4, [46,48) version = 1 on sm_100, [61,64) swizzle mode.
//   mode 2: 128-byte swizzle of 16-byte chunks, eight lines per 1024-byte atom (every bf16 tile, K-major tf32)
//   mode 1: 128-byte swizzle of 32-byte chunks, four lines per 512-byte atom -- the only layout the
//           tensor core accepts for MN-major 32-bit (tf32) operands
constexpr uint32_t kSwizzle128 = 2, kSwizzle128Base32 = 1;
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t leading_bytes, uint32_t stride_bytes, uint32_t mode) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((leading_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((stride_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)mode << 61;
  return d;
}

// Instruction descriptor for kind::f16 / kind::tf32 with f32 accumulation (PTX ISA, tcgen05 instruction
// descriptor): [4,6) D format (1 = f32), [7,10) A format, [10,13) B format (0 f16, 1 bf16, 2 tf32),
// bit 15 A major (0 = K, 1 = MN), bit 16 B major, [17,23) N >> 3, [24,29) M >> 4.
__host__ __device__ constexpr uint32_t make_instr_desc(uint32_t ab_format, uint32_t a_mn_major, uint32_t b_mn_major, uint32_t m, uint32_t n) {
  return (1u << 4) | (ab_format << 7) | (ab_format << 10) | (a_mn_major << 15) | (b_mn_major << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.  `accumulate` == 0 overwrites D.
__device__ __forceinline__ void mma_bf16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_tf32_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on `bar` once every tcgen05.mma issued so far by this thread has finished reading smem and
// writing TMEM.  Implies tcgen05.fence::before_thread_sync.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// One instruction across a CTA pair: M = 256 (128 rows per CTA), each CTA supplies its half of A's rows
// and half of B's columns from its own shared memory, each accumulates its 128 rows in its own TMEM.
// Issued by one thread of the leader CTA (cluster rank 0).
__device__ __forceinline__ void mma_pair_bf16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_pair_tf32_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the mbarrier at shared::cluster address `bar_addr` (either CTA of the pair) once every
// pair-MMA issued so far has completed in both CTAs.
__device__ __forceinline__ void mma_pair_commit(uint32_t bar_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_addr) : "memory");
}

// The same arrival delivered by one instruction to the mbarrier at this shared-memory offset in every CTA
// named by `cta_mask` (bit r = cluster rank r).  This is a barrier signal, not a data copy.
__device__ __forceinline__ void mma_pair_commit_both(uint64_t* bar, uint16_t cta_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(cta_mask) : "memory");
}

// Templated issue used by the mainloops: kPair selects cta_group::2, kTf32 the operand kind.  The
// accumulate flag is a register for the first K slice of a tile and the constant 1 for every other slice.
template <bool kPair, bool kTf32>
__device__ __forceinline__ void mma_issue(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  if constexpr (kPair) {
    if constexpr (kTf32) mma_pair_tf32_ss(tmem_d, desc_a, desc_b, idesc, accumulate);
    else mma_pair_bf16_ss(tmem_d, desc_a, desc_b, idesc, accumulate);
  } else {
    if constexpr (kTf32) mma_tf32_ss(tmem_d, desc_a, desc_b, idesc, accumulate);
    else mma_bf16_ss(tmem_d, desc_a, desc_b, idesc, accumulate);
  }
}

// ---- TMEM -> registers ------------------------------------------------------------------------------
// 32 lanes x 32 columns of 32-bit: thread t of the warp receives lane (base_lane + t), columns c..c+31.
// A warp may only touch the lane quarter (warp_id % 4) * 32 .. +31.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// bf16 round-to-nearest-even of an f32, the rounding grad's bf16 stores use
// (src/gpu/math/bf16.zig:1-5: (bits + 0x7FFF + ((bits >> 16) & 1)) >> 16, NaN handling included).
// f32 -> bf16, round to nearest even, by the conversion instruction.  On every finite value and on the
// infinities this is the integer formula (bits + 0x7FFF + ((bits >> 16) & 1)) >> 16; a NaN comes out as the
// canonical 0x7FFF where the formula would carry its payload into other bits.  Done with integer
// instructions the conversion was ~200 instructions per 32-column chunk, the largest part of a chunk's time.
__device__ __forceinline__ uint32_t bf16_bits(float x) {
  uint16_t h;
  asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(h) : "f"(x));
  return h;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
// f32 -> TF32 precision, round to nearest with ties away from zero (cvt.rna.tf32.f32), kept in an f32.
__device__ __forceinline__ float round_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}
__device__ __forceinline__ float bf16_to_f32(uint16_t h) { return __uint_as_float((uint32_t)h << 16); }
// relu(x * scale + shift) on a pair of bf16 values, each product-and-sum rounded once to bf16: the transform grad applies
// to an operand that stands for a normalised-and-rectified map (`affinePair`, src/gpu/device.zig:1604-1612).
__device__ __forceinline__ uint32_t affine_relu_bf16x2(uint32_t x2, uint32_t scale2, uint32_t shift2) {
  uint32_t out;
  asm("{\n"
      "fma.rn.bf16x2 %0, %1, %2, %3;\n"
      "max.bf16x2 %0, %0, %4;\n"
      "}\n"
      : "=r"(out)
      : "r"(x2), "r"(scale2), "r"(shift2), "r"(0u));
  return out;
}

}  // namespace gb
