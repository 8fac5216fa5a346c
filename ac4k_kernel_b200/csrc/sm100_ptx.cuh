// Thin inline-PTX wrappers for the sm_100a features the GEMM uses: mbarrier, TMA (tiled and
// linear bulk copies), tensor memory allocation, tcgen05.mma / cp / ld / commit / fences.
// Every wait is bounded: it gives up after kWaitTimeoutNs and reports through its return value.
#pragma once

#include <stdint.h>

namespace ac4k {
namespace ptx {

static constexpr unsigned long long kWaitTimeoutNs = 2000000000ull;   // 2 s

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long globaltimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ---- mbarrier ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false if the phase did not complete within `limit_ns` (the kernels pass the limit they were
// launched with: kWaitTimeoutNs unless a test build shortened it).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned long long limit_ns = kWaitTimeoutNs) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (globaltimer() - t0 > limit_ns) return false;
  }
}

// generic-proxy writes to shared memory -> visible to the async proxy (TMA, tcgen05.cp/mma)
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- TMA --------------------------------------------------------------------------------
// x is the innermost (byte) coordinate and must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void *tmap, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void *tmap, int x, int y, int z, int w, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(w), "r"(bar)
      : "memory");
}
// linear copy: src/dst 16-byte aligned, bytes a multiple of 16
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
// same, with the destination and the barrier named as shared::cta addresses (own CTA only)
__device__ __forceinline__ void bulk_load_1d_local(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d_local(uint32_t dst, const void *tmap, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
// Hint: bring the box into L2.  Returns no data, so it may be issued before griddepcontrol.wait: lines
// that an earlier kernel still writes are updated in L2, the point of coherence, like any others.
__device__ __forceinline__ void tma_prefetch_2d_if(uint32_t pred, const void *tmap, int x, int y) {
  asm volatile("{\n.reg .pred q;\nsetp.ne.b32 q, %3, 0;\n"
               "@q cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];\n}"
               ::"l"(tmap), "r"(x), "r"(y), "r"(pred) : "memory");
}
__device__ __forceinline__ void tma_prefetch_3d_if(uint32_t pred, const void *tmap, int x, int y, int z) {
  asm volatile("{\n.reg .pred q;\nsetp.ne.b32 q, %4, 0;\n"
               "@q cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];\n}"
               ::"l"(tmap), "r"(x), "r"(y), "r"(z), "r"(pred) : "memory");
}
// linear form of the same hint: `bytes` (multiple of 16) from a 16-byte aligned address
__device__ __forceinline__ void bulk_prefetch_l2_if(uint32_t pred, const void *src, uint32_t bytes) {
  asm volatile("{\n.reg .pred q;\nsetp.ne.b32 q, %2, 0;\n@q cp.async.bulk.prefetch.L2.global [%0], %1;\n}"
               ::"l"(src), "r"(bytes), "r"(pred) : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const void *tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ---- tensor memory ----------------------------------------------------------------------
// whole warp; writes the base address (lane 0, column c) to *dst_smem
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---- descriptors ------------------------------------------------------------------------
// Shared-memory matrix descriptor (K-major operand).  Fields: start address >> 4 in bits
// [0,14), leading-dimension byte offset >> 4 in [16,30), stride-dimension byte offset >> 4 in
// [32,46) (distance between 8-row groups), descriptor version 1 in [46,48), swizzle mode in
// [61,64) (0 none, 2 = 128-byte, 4 = 64-byte).
static constexpr uint32_t kSwizzleNone = 0, kSwizzle128B = 2, kSwizzle64B = 4;
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                   uint32_t swizzle) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)(swizzle & 7) << 61;
  return d;
}

// Instruction descriptor of kind::mxf4nvf4 with block scaling: e2m1 A and B (format code 1 in
// [7,10) and [10,13)), both K-major (bits 15, 16 clear), N >> 3 in [17,23), scale format
// UE4M3 (bit 23 clear), M >> 4 in [24,29), scale-factor byte ids 0 (4 scales per 32-bit
// column), K = 64 (bit 31 clear).
__host__ __device__ constexpr uint32_t make_idesc_mxf4nvf4(int m, int n) {
  return (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ---- tcgen05 ----------------------------------------------------------------------------
// D[tmem] (+)= A[smem] * B[smem]^T with per-16-element block scales taken from tensor memory.
__device__ __forceinline__ void mma_mxf4nvf4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %6, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
      : "memory");
}
// 32 rows x 16 bytes of shared memory -> 4 columns of tensor memory, replicated to the four
// 32-lane quarters.
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// arrive on an mbarrier once all tcgen05 operations issued so far by this thread are done
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// each lane reads 32 consecutive 32-bit columns of its own tensor-memory lane
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
// each lane writes N consecutive 32-bit columns of its own tensor-memory lane
__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
        "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
        "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x64(uint32_t taddr, const uint32_t (&v)[64]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x64.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63, %64};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31]), "r"(v[32]), "r"(v[33]), "r"(v[34]), "r"(v[35]), "r"(v[36]), "r"(v[37]), "r"(v[38]), "r"(v[39]), "r"(v[40]), "r"(v[41]), "r"(v[42]), "r"(v[43]), "r"(v[44]), "r"(v[45]), "r"(v[46]), "r"(v[47]), "r"(v[48]), "r"(v[49]), "r"(v[50]), "r"(v[51]), "r"(v[52]), "r"(v[53]), "r"(v[54]), "r"(v[55]), "r"(v[56]), "r"(v[57]), "r"(v[58]), "r"(v[59]), "r"(v[60]), "r"(v[61]), "r"(v[62]), "r"(v[63])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// Load + wait, with the loaded registers pinned behind the wait.  tcgen05.ld writes its registers
// asynchronously and only tcgen05.wait::ld makes them valid, but the wait has no register operands,
// so the compiler is otherwise free to schedule arithmetic on `v` between the two (observed: rare
// blocks of wrong output).  The empty volatile asm statements make every later use depend on a
// statement that is ordered after the wait.
__device__ __forceinline__ void tmem_ld_32x32b_x32_sync(uint32_t taddr, uint32_t (&v)[32]) {
  tmem_ld_32x32b_x32(taddr, v);
  tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < 32; ++i) asm volatile("" : "+r"(v[i]) : : "memory");
}


__device__ __forceinline__ void tmem_ld_32x32b_x64_sync(uint32_t taddr, uint32_t (&v)[64]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31]), "=r"(v[32]), "=r"(v[33]), "=r"(v[34]), "=r"(v[35]), "=r"(v[36]), "=r"(v[37]), "=r"(v[38]), "=r"(v[39]), "=r"(v[40]), "=r"(v[41]), "=r"(v[42]), "=r"(v[43]), "=r"(v[44]), "=r"(v[45]), "=r"(v[46]), "=r"(v[47]), "=r"(v[48]), "=r"(v[49]), "=r"(v[50]), "=r"(v[51]), "=r"(v[52]), "=r"(v[53]), "=r"(v[54]), "=r"(v[55]), "=r"(v[56]), "=r"(v[57]), "=r"(v[58]), "=r"(v[59]), "=r"(v[60]), "=r"(v[61]), "=r"(v[62]), "=r"(v[63])
      : "r"(taddr)
      : "memory");
  tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < 64; ++i) asm volatile("" : "+r"(v[i]) : : "memory");
}

// tcgen05.ld without the wait, for several loads in flight behind one tcgen05.wait::ld; the caller
// pins the registers with tmem_pin() after the wait (see tmem_ld_32x32b_x32_sync).
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x64(uint32_t taddr, uint32_t (&v)[64]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31]), "=r"(v[32]), "=r"(v[33]), "=r"(v[34]), "=r"(v[35]), "=r"(v[36]), "=r"(v[37]), "=r"(v[38]), "=r"(v[39]), "=r"(v[40]), "=r"(v[41]), "=r"(v[42]), "=r"(v[43]), "=r"(v[44]), "=r"(v[45]), "=r"(v[46]), "=r"(v[47]), "=r"(v[48]), "=r"(v[49]), "=r"(v[50]), "=r"(v[51]), "=r"(v[52]), "=r"(v[53]), "=r"(v[54]), "=r"(v[55]), "=r"(v[56]), "=r"(v[57]), "=r"(v[58]), "=r"(v[59]), "=r"(v[60]), "=r"(v[61]), "=r"(v[62]), "=r"(v[63])
      : "r"(taddr)
      : "memory");
}
template <int N>
__device__ __forceinline__ void tmem_pin(uint32_t (&v)[N]) {
#pragma unroll
  for (int i = 0; i < N; ++i) asm volatile("" : "+r"(v[i]) : : "memory");
}

__device__ __forceinline__ uint32_t ld_shared_volatile(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.volatile.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void st_shared_v4f(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cta.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ float4 ld_shared_v4f(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cta.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ float2 ld_shared_v2f(uint32_t addr) {
  float2 v;
  asm volatile("ld.shared::cta.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void st_shared_release(uint32_t addr, uint32_t v) {
  asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}

// (a0 * s, a1 * s) in fp32, round to nearest, packed to two bf16 / fp16 (element 0 in the low half)
__device__ __forceinline__ uint32_t scale_pack_bf16x2(uint32_t a0, uint32_t a1, float s) {
  uint32_t out;
  asm("{\n.reg .b64 p, ss;\n.reg .f32 x, y;\n"
      "mov.b64 p, {%1, %2};\n mov.b64 ss, {%3, %3};\n mul.rn.f32x2 p, p, ss;\n mov.b64 {x, y}, p;\n"
      "cvt.rn.bf16x2.f32 %0, y, x;\n}"
      : "=r"(out) : "r"(a0), "r"(a1), "f"(s));
  return out;
}
// ((a0 * s) + b0, (a1 * s) + b1): product and sum each rounded to nearest in fp32, packed to bf16 / fp16
__device__ __forceinline__ uint32_t scale_bias_pack_bf16x2(uint32_t a0, uint32_t a1, float s, float b0, float b1) {
  uint32_t out;
  asm("{\n.reg .b64 p, ss, bb;\n.reg .f32 x, y;\n"
      "mov.b64 p, {%1, %2};\n mov.b64 ss, {%3, %3};\n mov.b64 bb, {%4, %5};\n"
      "mul.rn.f32x2 p, p, ss;\n add.rn.f32x2 p, p, bb;\n mov.b64 {x, y}, p;\n"
      "cvt.rn.bf16x2.f32 %0, y, x;\n}"
      : "=r"(out) : "r"(a0), "r"(a1), "f"(s), "f"(b0), "f"(b1));
  return out;
}
__device__ __forceinline__ uint32_t scale_bias_pack_f16x2(uint32_t a0, uint32_t a1, float s, float b0, float b1) {
  uint32_t out;
  asm("{\n.reg .b64 p, ss, bb;\n.reg .f32 x, y;\n"
      "mov.b64 p, {%1, %2};\n mov.b64 ss, {%3, %3};\n mov.b64 bb, {%4, %5};\n"
      "mul.rn.f32x2 p, p, ss;\n add.rn.f32x2 p, p, bb;\n mov.b64 {x, y}, p;\n"
      "cvt.rn.f16x2.f32 %0, y, x;\n}"
      : "=r"(out) : "r"(a0), "r"(a1), "f"(s), "f"(b0), "f"(b1));
  return out;
}
__device__ __forceinline__ uint32_t scale_pack_f16x2(uint32_t a0, uint32_t a1, float s) {
  uint32_t out;
  asm("{\n.reg .b64 p, ss;\n.reg .f32 x, y;\n"
      "mov.b64 p, {%1, %2};\n mov.b64 ss, {%3, %3};\n mul.rn.f32x2 p, p, ss;\n mov.b64 {x, y}, p;\n"
      "cvt.rn.f16x2.f32 %0, y, x;\n}"
      : "=r"(out) : "r"(a0), "r"(a1), "f"(s));
  return out;
}

// 32-byte global store (one full sector per lane)
__device__ __forceinline__ void st_global_v8(void *p, uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t e,
                                             uint32_t f, uint32_t g, uint32_t h) {
  asm volatile("st.global.L1::no_allocate.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d), "r"(e), "r"(f), "r"(g), "r"(h)
               : "memory");
}

// 16-byte global load served by L2 (never by this SM's L1, which may hold a stale line)
__device__ __forceinline__ uint4 ld_global_cg_v4(const void *p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
// 16-byte global store without L1 allocation (used for peer memory)
__device__ __forceinline__ void st_global_v4(void *p, uint4 v) {
  asm volatile("st.global.L1::no_allocate.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// ---- CTA pairs (cta_group::2) and clusters ----------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
// 16-byte store into the shared memory of a CTA of this cluster (address from map_to_cta)
__device__ __forceinline__ void st_shared_cluster_v4(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}
// cluster barrier that only holds the CTAs back until all have arrived (no memory ordering of its own)
__device__ __forceinline__ void cluster_sync_relaxed() {
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
}
// arrive on an mbarrier given by a shared::cluster address (own or peer CTA).  Default semantics
// (release at CTA scope): the cluster-scope release form was measured at ~0.7 us per arrive,
// and the data handed over here (tensor memory) is ordered by the tcgen05 fences instead.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void named_barrier_sync(uint32_t id, uint32_t nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
// TMA load whose completion is signalled on an mbarrier that may live in the peer CTA of the pair
// (shared::cluster addresses for both the destination and the barrier)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const void *tmap, int x, int y, uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(bar_cluster_addr)
      : "memory");
}
// TMA store shared -> global (tiled, clipped at the tensor bounds); x in elements of the map
__device__ __forceinline__ void tma_store_2d(const void *tmap, int x, int y, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];"
               ::"l"(tmap), "r"(x), "r"(y), "r"(src)
               : "memory");
}
__device__ __forceinline__ void tma_store_3d(const void *tmap, int x, int y, int z, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];"
               ::"l"(tmap), "r"(x), "r"(y), "r"(z), "r"(src)
               : "memory");
}
// same, with an L2 cache policy for the written lines (from make_policy_evict_first / _last)
__device__ __forceinline__ void tma_store_2d_hint(const void *tmap, int x, int y, uint32_t src, uint64_t policy) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group.L2::cache_hint [%0, {%1, %2}], [%3], %4;"
               ::"l"(tmap), "r"(x), "r"(y), "r"(src), "l"(policy)
               : "memory");
}
__device__ __forceinline__ uint64_t make_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t make_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_group_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void bulk_wait_group0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// one MMA over both CTAs of the pair: M = 256 (128 rows per CTA), B halves read from both CTAs
__device__ __forceinline__ void mma_mxf4nvf4_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                  uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %6, 0;\n"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
      : "memory");
}
// completion of this thread's earlier tcgen05 work -> one arrival on the mbarrier at this
// shared-memory offset in every CTA of `cta_mask` (both CTAs of the pair: 3).  This is the
// commit's own arrival fan-out, not a multicast load.
__device__ __forceinline__ void tc_commit_pair_both(uint32_t bar, uint16_t cta_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(cta_mask)
               : "memory");
}
// completion of this thread's earlier tcgen05 work -> one arrival on an mbarrier given by a
// shared::cluster address (own or peer CTA)
__device__ __forceinline__ void tc_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
               : "memory");
}

// ---- warp-wide issue ----------------------------------------------------------------------
// A role that issues tcgen05 / TMA instructions runs with its whole warp converged and gives every
// such instruction a predicate that is true in one elected lane.  Measured on a B200: issued from
// inside an `if (lane == 0)` branch a tcgen05.mma / cp / commit costs the issuing thread 70 - 110
// cycles each (a stage of 12 cp + 4 mma + 1 commit: 1 080 cycles); issued predicated from a converged
// warp the same stage costs 330 cycles, because addresses and descriptors stay in uniform registers.
__device__ __forceinline__ uint32_t elect_one() {
  uint32_t pred;
  asm volatile("{\n.reg .pred P;\nelect.sync _|P, 0xffffffff;\nselp.u32 %0, 1, 0, P;\n}" : "=r"(pred));
  return pred;
}
__device__ __forceinline__ bool warp_all(bool v) { return __all_sync(0xffffffffu, v); }

__device__ __forceinline__ void mbar_arrive_expect_tx_if(uint32_t pred, uint32_t bar, uint32_t bytes) {
  asm volatile("{\n.reg .pred q;\nsetp.ne.b32 q, %2, 0;\n@q mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n}"
               ::"r"(bar), "r"(bytes), "r"(pred) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster_if(uint32_t pred, uint32_t bar_cluster_addr) {
  asm volatile("{\n.reg .pred q;\nsetp.ne.b32 q, %1, 0;\n@q mbarrier.arrive.shared::cluster.b64 _, [%0];\n}"
               ::"r"(bar_cluster_addr), "r"(pred) : "memory");
}
__device__ __forceinline__ void tma_load_2d_if(uint32_t pred, uint32_t dst, const void *tmap, int x, int y, uint32_t bar) {
  asm volatile(
      "{\n.reg .pred q;\nsetp.ne.b32 q, %5, 0;\n"
      "@q cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n}"
      ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(bar), "r"(pred)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair_if(uint32_t pred, uint32_t dst, const void *tmap, int x, int y,
                                                    uint32_t bar_cluster_addr) {
  asm volatile(
      "{\n.reg .pred q;\nsetp.ne.b32 q, %5, 0;\n"
      "@q cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n}"
      ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(bar_cluster_addr), "r"(pred)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair_if(uint32_t pred, uint32_t dst, const void *tmap, int x, int y, int z,
                                                    uint32_t bar_cluster_addr) {
  asm volatile(
      "{\n.reg .pred q;\nsetp.ne.b32 q, %6, 0;\n"
      "@q cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n}"
      ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(bar_cluster_addr), "r"(pred)
      : "memory");
}
__device__ __forceinline__ void bulk_load_1d_if(uint32_t pred, uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "{\n.reg .pred q;\nsetp.ne.b32 q, %4, 0;\n"
      "@q cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n}"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "r"(pred)
      : "memory");
}
__device__ __forceinline__ void mma_mxf4nvf4_if(uint32_t pred, uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p, q;\nsetp.ne.b32 p, %6, 0;\nsetp.ne.b32 q, %7, 0;\n"
      "@q tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate), "r"(pred)
      : "memory");
}
__device__ __forceinline__ void mma_mxf4nvf4_pair_if(uint32_t pred, uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                     uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p, q;\nsetp.ne.b32 p, %6, 0;\nsetp.ne.b32 q, %7, 0;\n"
      "@q tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate), "r"(pred)
      : "memory");
}
// 32 rows x 16 bytes of shared memory -> 4 columns of tensor memory, replicated to the four 32-lane
// quarters.  The pair form copies in both CTAs, each from its own shared memory at the same offset
// into its own tensor memory.  Executes in issue order with the MMAs of the same thread and overlaps
// them: (12 cp + 4 MMA of 128 x 256 x 64) run in 523 cycles against 520 for the MMAs alone.
__device__ __forceinline__ void tmem_cp_32x128b_warpx4_if(uint32_t pred, uint32_t taddr, uint64_t sdesc) {
  asm volatile("{\n.reg .pred q;\nsetp.ne.b32 q, %2, 0;\n@q tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;\n}"
               ::"r"(taddr), "l"(sdesc), "r"(pred) : "memory");
}
__device__ __forceinline__ void tmem_cp_32x128b_warpx4_pair_if(uint32_t pred, uint32_t taddr, uint64_t sdesc) {
  asm volatile("{\n.reg .pred q;\nsetp.ne.b32 q, %2, 0;\n@q tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;\n}"
               ::"r"(taddr), "l"(sdesc), "r"(pred) : "memory");
}
__device__ __forceinline__ void tc_commit_if(uint32_t pred, uint32_t bar) {
  asm volatile("{\n.reg .pred q;\nsetp.ne.b32 q, %1, 0;\n"
               "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n}"
               ::"r"(bar), "r"(pred) : "memory");
}
__device__ __forceinline__ void tc_commit_pair_both_if(uint32_t pred, uint32_t bar, uint16_t cta_mask) {
  asm volatile("{\n.reg .pred q;\nsetp.ne.b32 q, %2, 0;\n"
               "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n}"
               ::"r"(bar), "h"(cta_mask), "r"(pred)
               : "memory");
}
__device__ __forceinline__ void st_shared_v4u(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared::cta.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

}  // namespace ptx
}  // namespace ac4k
