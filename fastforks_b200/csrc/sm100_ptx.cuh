// Thin inline-PTX wrappers for the Blackwell (sm_100a) features the attention kernels use:
// mbarrier, TMA tensor copies (never with cluster multicast), tensor memory (TMEM) management,
// tcgen05 MMA issue / commit, TMEM loads and stores.
//
// Every wait in here is bounded: `mbar_wait` gives up after a wall-clock limit and reports failure
// instead of spinning for ever, so a protocol bug ends as an error status, not as a hung GPU.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Hands registers from one warpgroup to another: every warp of a warpgroup must execute the same call.
template <int REGS>
__device__ __forceinline__ void reg_alloc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS));
}
template <int REGS>
__device__ __forceinline__ void reg_dealloc() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS));
}

// ---------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// Non-blocking probe: true when the phase with the given parity has completed.
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// Wall-clock limit of one wait. A healthy launch finishes every wait in microseconds.
#ifndef B200_WAIT_LIMIT_NS
#define B200_WAIT_LIMIT_NS 1000000000ull
#endif

// Waits for the phase with the given parity to complete. Returns false when the limit ran out or
// when another thread of the CTA has already raised `*abort_flag` (shared memory).
// The wall clock is only consulted after a long run of failed polls (each try_wait already sleeps in
// hardware for a while), so a wait that succeeds quickly costs a handful of instructions.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag) {
#pragma unroll 1
  for (uint32_t polls = 0; polls < 4096; ++polls)
    if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t polls = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++polls & 0xff) == 0) {
      if (*abort_flag != 0) return false;
      if (global_timer_ns() - t0 > B200_WAIT_LIMIT_NS) return false;
    }
  }
}

// Wait of a whole warp on a barrier whose phase has, as a rule, completed long ago: one poll and no vote on that
// path. Returns false for a lane whose wait ran out; the caller collects that per lane and votes once per step.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag) {
  bool done = mbar_try_wait(bar, parity);
  if (!done) done = mbar_wait(bar, parity, abort_flag);
  __syncwarp();
  return done;
}

// Second half of a wait whose first test was issued early (mbar_test_wait, its latency hidden behind other work):
// `early` is that test's result; only a lane that saw the phase still pending waits now.
__device__ __forceinline__ bool mbar_wait_warp_after(bool early, uint64_t* bar, uint32_t parity,
                                                      volatile uint32_t* abort_flag) {
  bool done = early;
  if (!done) done = mbar_wait(bar, parity, abort_flag);
  __syncwarp();
  return done;
}

// The same for the loader thread: it sleeps between polls so that its spinning does not take issue slots from the
// softmax warps that share its SM sub-partition. The sleep costs some 300 clocks of wake-up latency (80 without),
// which is off the critical path here: loads run several tiles ahead. The MMA issuers use mbar_wait.
__device__ __forceinline__ bool mbar_wait_relaxed(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
#pragma unroll 1
  for (uint32_t polls = 0; polls < 4096; ++polls) {
    __nanosleep(64);
    if (mbar_try_wait(bar, parity)) return true;
  }
  const uint64_t t0 = global_timer_ns();
  uint32_t polls = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    __nanosleep(256);
    if ((++polls & 0xff) == 0) {
      if (*abort_flag != 0) return false;
      if (global_timer_ns() - t0 > B200_WAIT_LIMIT_NS) return false;
    }
  }
}

// Acquire load of a word another CTA of the grid may have written with a release / fenced atomic.
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* word) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(word) : "memory");
  return v;
}

// ---------------------------------------------------------------------------------------------
// Proxy / tcgen05 fences
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// TMA (tiled tensor copies through a CUtensorMap). Loads signal an mbarrier with their byte count.
// x is the innermost coordinate and must keep the copy 16-byte aligned.
// ---------------------------------------------------------------------------------------------
// Wait until the grids this one depends on (the kernel launched before it in the stream, when this one was launched
// with programmatic stream serialisation) have completed and flushed their memory operations.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y,
                                            int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z),
        "r"(w)
      : "memory");
}

__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, const void* smem_src, int x, int y, int z,
                                             int w) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               :
               : "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z), "r"(w)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until at most `N` of this thread's store groups still read shared memory.
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------------------------------------
// Tensor memory
// ---------------------------------------------------------------------------------------------
// One full warp allocates `cols` (power of two, 32..512) columns; the base address lands in *slot.
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

// ---------------------------------------------------------------------------------------------
// UMMA descriptors
// ---------------------------------------------------------------------------------------------
// Shared-memory matrix descriptor for a tile stored as 128-byte rows with the 128-byte swizzle
// (what a TMA load with CU_TENSOR_MAP_SWIZZLE_128B of a 64-element 16-bit inner box writes).
// `sbo_bytes` is the distance between consecutive 8-row groups (1024 for a dense tile),
// `lbo_bytes` the distance between 64-element columns blocks for MN-major operands wider than 64.
__device__ __forceinline__ uint64_t umma_smem_desc_sw128(uint32_t smem_addr, uint32_t sbo_bytes,
                                                         uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);            // bits  0..13 start address
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;       // bits 16..29 leading byte offset
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;       // bits 32..45 stride byte offset
  d |= static_cast<uint64_t>(1) << 46;                               // bits 46..47 descriptor version (sm_100)
  d |= static_cast<uint64_t>(2) << 61;                               // bits 61..63 layout: 128-byte swizzle
  return d;
}

enum : uint32_t { UMMA_F16 = 0, UMMA_BF16 = 1 };

// Instruction descriptor of tcgen05.mma.kind::f16 with fp32 accumulation.
// a_mn / b_mn: 1 when that operand is MN-major (its M/N index is the contiguous one in memory).
__host__ __device__ constexpr uint32_t umma_idesc_f16(uint32_t ab_format, uint32_t m, uint32_t n, uint32_t a_mn,
                                                      uint32_t b_mn) {
  return (1u << 4)               // D format: F32
         | (ab_format << 7)      // A format
         | (ab_format << 10)     // B format
         | (a_mn << 15) | (b_mn << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]; issued by ONE thread. A is K-major: lane = row, 32-bit column = two K elements.
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Makes `bar` (count 1) complete once every tcgen05.mma this thread issued before has finished.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// ---------------------------------------------------------------------------------------------
// TMEM <-> registers. Warp w of a warpgroup reaches lanes 32*(w%4) .. 32*(w%4)+31; with the 32x32b
// shape thread i of the warp owns lane 32*(w%4)+i and receives consecutive 32-bit columns.
// Each load waits for its data inside the same asm block, so results are valid on return.
// ---------------------------------------------------------------------------------------------
#define B200_R4(v, i) "=r"(v[i]), "=r"(v[i + 1]), "=r"(v[i + 2]), "=r"(v[i + 3])
#define B200_R16(v, i) B200_R4(v, i), B200_R4(v, i + 4), B200_R4(v, i + 8), B200_R4(v, i + 12)
#define B200_W4(v, i) "r"(v[i]), "r"(v[i + 1]), "r"(v[i + 2]), "r"(v[i + 3])
#define B200_W16(v, i) B200_W4(v, i), B200_W4(v, i + 4), B200_W4(v, i + 8), B200_W4(v, i + 12)

__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n\t"
      "tcgen05.wait::ld.sync.aligned;\n"
      : B200_R16(v, 0)
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n\t"
      "tcgen05.wait::ld.sync.aligned;\n"
      : B200_R16(v, 0), B200_R16(v, 16)
      : "r"(taddr)
      : "memory");
}

// Two 32-column loads in flight, one wait.
__device__ __forceinline__ void tmem_ld_x64(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%64];\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, "
      "%48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%65];\n\t"
      "tcgen05.wait::ld.sync.aligned;\n"
      : B200_R16(v, 0), B200_R16(v, 16), B200_R16(v, 32), B200_R16(v, 48)
      : "r"(taddr), "r"(taddr + 32)
      : "memory");
}

// Asynchronous load: the registers are valid only after tmem_ld_wait_pin() on the same registers.
__device__ __forceinline__ void tmem_ld_x32_nowait(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : B200_R16(v, 0), B200_R16(v, 16)
      : "r"(taddr)
      : "memory");
}

#define B200_P4(v, i) "+r"(v[i]), "+r"(v[i + 1]), "+r"(v[i + 2]), "+r"(v[i + 3])
#define B200_P16(v, i) B200_P4(v, i), B200_P4(v, i + 4), B200_P4(v, i + 8), B200_P4(v, i + 12)

// Waits for all of this thread's tensor-memory loads. The 32 registers are routed through the instruction so that
// no use of them is scheduled before the wait; call tmem_ld_pin() for further registers of the same batch.
__device__ __forceinline__ void tmem_ld_wait_pin(uint32_t* v) {
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" : B200_P16(v, 0), B200_P16(v, 16) : : "memory");
}
__device__ __forceinline__ void tmem_ld_pin(uint32_t* v) {
  asm volatile("" : B200_P16(v, 0), B200_P16(v, 16) : : "memory");
}

__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};\n"
      :
      : "r"(taddr), B200_W16(v, 0)
      : "memory");
}

__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
      :
      : "r"(taddr), B200_W16(v, 0), B200_W16(v, 16)
      : "memory");
}

// 128 columns with one instruction. It needs 128 result registers at once: a kernel whose launch bound allows fewer
// than about 146 registers per thread does not assemble with it, whatever setmaxnreg raises the budget to later.
__device__ __forceinline__ void tmem_ld_x128(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x128.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63, %64, %65, %66, %67, %68, %69, %70, %71, %72, %73, %74, %75, %76, %77, %78, %79, %80, %81, %82, %83, %84, %85, %86, %87, %88, %89, %90, %91, %92, %93, %94, %95, %96, %97, %98, %99, %100, %101, %102, %103, %104, %105, %106, %107, %108, %109, %110, %111, %112, %113, %114, %115, %116, %117, %118, %119, %120, %121, %122, %123, %124, %125, %126, %127}, [%128];\n\t"
      "tcgen05.wait::ld.sync.aligned;\n"
      : B200_R16(v, 0), B200_R16(v, 16), B200_R16(v, 32), B200_R16(v, 48), B200_R16(v, 64), B200_R16(v, 80), B200_R16(v, 96), B200_R16(v, 112)
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_x64(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x64.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63, %64};\n"
      :
      : "r"(taddr), B200_W16(v, 0), B200_W16(v, 16), B200_W16(v, 32), B200_W16(v, 48)
      : "memory");
}

__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

}  // namespace b200
