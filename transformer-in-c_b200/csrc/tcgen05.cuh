// PTX wrappers shared by the tensor-core kernels of this library (sm_100a):
// mbarriers with bounded waits, TMA tile copies, tcgen05 MMA / tensor-memory
// loads and stores, and the shared-memory operand descriptor.
#pragma once

#include <cuda.h>
#include <cstdint>
#include <cuda_runtime.h>

namespace vitb200 {
namespace tc {

constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s

__device__ __forceinline__ uint32_t smem_address(const void *pointer) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(pointer));
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbarrier_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_address(bar)),
                 "r"(count));
}

__device__ __forceinline__ void mbarrier_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(
                     smem_address(bar)),
                 "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbarrier_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_address(bar))
                 : "memory");
}

__device__ __forceinline__ bool mbarrier_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(done)
        : "r"(smem_address(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

// Returns false if the phase did not complete within kWaitLimitNs.
__device__ __forceinline__ bool mbarrier_wait(uint64_t *bar, uint32_t parity) {
    if (mbarrier_try_wait(bar, parity)) {
        return true;
    }
    const unsigned long long start = global_timer_ns();
    while (!mbarrier_try_wait(bar, parity)) {
        if (global_timer_ns() - start > kWaitLimitNs) {
            return false;
        }
    }
    return true;
}

__device__ __forceinline__ void tma_load_2d(void *smem, const CUtensorMap *map,
                                            int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3}], [%4];" ::"r"(smem_address(smem)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y),
        "r"(smem_address(bar))
        : "memory");
}

__device__ __forceinline__ void tma_load_3d(void *smem, const CUtensorMap *map,
                                            int x, int y, int z, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(smem_address(smem)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z),
        "r"(smem_address(bar))
        : "memory");
}

__device__ __forceinline__ void tma_store_2d(const void *smem,
                                             const CUtensorMap *map, int x,
                                             int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::
            "l"(reinterpret_cast<uint64_t>(map)),
        "r"(smem_address(smem)), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void tma_store_3d(const void *smem,
                                             const CUtensorMap *map, int x,
                                             int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.global.shared::cta.bulk_group"
        " [%0, {%2, %3, %4}], [%1];" ::"l"(reinterpret_cast<uint64_t>(map)),
        "r"(smem_address(smem)), "r"(x), "r"(y), "r"(z)
        : "memory");
}

__device__ __forceinline__ void tma_reduce_add_2d(const void *smem,
                                                  const CUtensorMap *map, int x,
                                                  int y) {
    asm volatile(
        "cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group"
        " [%0, {%2, %3}], [%1];" ::"l"(reinterpret_cast<uint64_t>(map)),
        "r"(smem_address(smem)), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void tma_reduce_add_3d(const void *smem,
                                                  const CUtensorMap *map, int x,
                                                  int y, int z) {
    asm volatile(
        "cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.bulk_group"
        " [%0, {%2, %3, %4}], [%1];" ::"l"(reinterpret_cast<uint64_t>(map)),
        "r"(smem_address(smem)), "r"(x), "r"(y), "r"(z)
        : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tcgen05_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tcgen05_commit(uint64_t *bar) {
    asm volatile(
        "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::
            "r"(smem_address(bar))
        : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], TF32 operands, FP32 accumulation.
__device__ __forceinline__ void tcgen05_mma_tf32(uint32_t tmem_d, uint64_t desc_a,
                                                 uint64_t desc_b, uint32_t idesc,
                                                 uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// The same, issued only by lanes whose `issue` flag is set.  The whole warp
// executes the statement (no branch around it), so operands that every lane
// computes alike stay in uniform registers, which is where the instruction
// reads them from.
__device__ __forceinline__ void tcgen05_mma_tf32_if(uint32_t issue, uint32_t tmem_d,
                                                    uint64_t desc_a, uint64_t desc_b,
                                                    uint32_t idesc,
                                                    uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.ne.b32 q, %5, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(issue)
        : "memory");
}

// A operand in tensor memory: 128 lanes x 8 columns of 32-bit cells per
// instruction, reduction index along the columns.
__device__ __forceinline__ void tcgen05_mma_tf32_tmem_a_if(uint32_t issue,
                                                           uint32_t tmem_d,
                                                           uint32_t tmem_a,
                                                           uint64_t desc_b,
                                                           uint32_t idesc,
                                                           uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.ne.b32 q, %5, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t"
        "}" ::"r"(tmem_d),
        "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(issue)
        : "memory");
}

__device__ __forceinline__ void tcgen05_commit_if(uint32_t issue, uint64_t *bar) {
    asm volatile(
        "{\n\t"
        ".reg .pred q;\n\t"
        "setp.ne.b32 q, %1, 0;\n\t"
        "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
        "}" ::"r"(smem_address(bar)),
        "r"(issue)
        : "memory");
}

// Lane i of the warp receives columns [column, column + 32) of tensor-memory
// lane (address lane field) + i.  Returns after the values have arrived.
__device__ __forceinline__ void tcgen05_load_32(uint32_t tmem_address,
                                                uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32"
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15,"
        " %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29,"
        " %30, %31}, [%32];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),
          "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
          "=r"(r[31])
        : "r"(tmem_address)
        : "memory");
}

// The reverse: lane i writes its 32 values to columns [column, column + 32)
// of its tensor-memory lane.  Asynchronous; tcgen05_wait_store() completes it.
__device__ __forceinline__ void tcgen05_store_32(uint32_t tmem_address,
                                                 const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16,"
        " %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30,"
        " %31, %32};" ::"r"(tmem_address),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]),
        "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
        "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
        "r"(r[30]), "r"(r[31])
        : "memory");
}

// 64 consecutive columns at once (one instruction, one wait).
__device__ __forceinline__ void tcgen05_load_64(uint32_t tmem_address,
                                                uint32_t (&r)[64]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 {"
        "%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16,"
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31,"
        "%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46,"
        "%47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61,"
        "%62, %63"
        "}, [%64];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),
          "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
          "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]),
          "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
          "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]),
          "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]),
          "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]),
          "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]),
          "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]),
          "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
        : "r"(tmem_address)
        : "memory");
}

__device__ __forceinline__ void tcgen05_store_64(uint32_t tmem_address,
                                                 const uint32_t (&r)[64]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x64.b32 [%64], {"
        "%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16,"
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31,"
        "%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46,"
        "%47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61,"
        "%62, %63"
        "};"
        :
        : "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
          "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]),
          "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
          "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
          "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
          "r"(r[31]), "r"(r[32]), "r"(r[33]), "r"(r[34]), "r"(r[35]), "r"(r[36]),
          "r"(r[37]), "r"(r[38]), "r"(r[39]), "r"(r[40]), "r"(r[41]), "r"(r[42]),
          "r"(r[43]), "r"(r[44]), "r"(r[45]), "r"(r[46]), "r"(r[47]), "r"(r[48]),
          "r"(r[49]), "r"(r[50]), "r"(r[51]), "r"(r[52]), "r"(r[53]), "r"(r[54]),
          "r"(r[55]), "r"(r[56]), "r"(r[57]), "r"(r[58]), "r"(r[59]), "r"(r[60]),
          "r"(r[61]), "r"(r[62]), "r"(r[63]),
          "r"(tmem_address)
        : "memory");
}

// Two 32-column blocks (different addresses) with one wait, so that the two
// reads overlap.
__device__ __forceinline__ void tcgen05_load_32_pair(uint32_t address_a,
                                                     uint32_t address_b,
                                                     uint32_t (&a)[32],
                                                     uint32_t (&b)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {"
        "%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16,"
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31"
        "}, [%64];\n\t"
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {"
        "%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46,"
        "%47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61,"
        "%62, %63"
        "}, [%65];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]), "=r"(a[4]), "=r"(a[5]),
          "=r"(a[6]), "=r"(a[7]), "=r"(a[8]), "=r"(a[9]), "=r"(a[10]), "=r"(a[11]),
          "=r"(a[12]), "=r"(a[13]), "=r"(a[14]), "=r"(a[15]), "=r"(a[16]), "=r"(a[17]),
          "=r"(a[18]), "=r"(a[19]), "=r"(a[20]), "=r"(a[21]), "=r"(a[22]), "=r"(a[23]),
          "=r"(a[24]), "=r"(a[25]), "=r"(a[26]), "=r"(a[27]), "=r"(a[28]), "=r"(a[29]),
          "=r"(a[30]), "=r"(a[31]),
          "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]), "=r"(b[4]), "=r"(b[5]),
          "=r"(b[6]), "=r"(b[7]), "=r"(b[8]), "=r"(b[9]), "=r"(b[10]), "=r"(b[11]),
          "=r"(b[12]), "=r"(b[13]), "=r"(b[14]), "=r"(b[15]), "=r"(b[16]), "=r"(b[17]),
          "=r"(b[18]), "=r"(b[19]), "=r"(b[20]), "=r"(b[21]), "=r"(b[22]), "=r"(b[23]),
          "=r"(b[24]), "=r"(b[25]), "=r"(b[26]), "=r"(b[27]), "=r"(b[28]), "=r"(b[29]),
          "=r"(b[30]), "=r"(b[31])
        : "r"(address_a), "r"(address_b)
        : "memory");
}

__device__ __forceinline__ void tcgen05_wait_store() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_allocate(uint32_t *slot, uint32_t columns) {
    asm volatile(
        "tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
            smem_address(slot)),
        "r"(columns)
        : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::
                     : "memory");
}

__device__ __forceinline__ void tmem_free(uint32_t base, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base),
                 "r"(columns)
                 : "memory");
}

// FP32 -> TF32 (10 mantissa bits), round to nearest, ties away from zero.
__device__ __forceinline__ uint32_t round_tf32(float x) {
    uint32_t y;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float exp2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Shared-memory operand descriptor with the Blackwell version field.  Offsets
// are in bytes; the hardware fields drop the low four bits.  Layout types:
// 2 = 128-byte swizzle of 16-byte chunks (K-major operands), 1 = 128-byte
// swizzle of 32-byte chunks, the only layout tcgen05 accepts for 32-bit
// operands whose output index is the contiguous one.
constexpr uint32_t kLayoutSwizzle128 = 2;
constexpr uint32_t kLayoutSwizzle128Base32 = 1;
__device__ __forceinline__ uint64_t operand_descriptor(uint32_t smem_byte_address,
                                                       uint32_t leading_bytes,
                                                       uint32_t stride_bytes,
                                                       uint32_t layout_type) {
    uint64_t desc = 0;
    desc |= uint64_t((smem_byte_address >> 4) & 0x3fff);
    desc |= uint64_t((leading_bytes >> 4) & 0x3fff) << 16;
    desc |= uint64_t((stride_bytes >> 4) & 0x3fff) << 32;
    desc |= uint64_t(1) << 46;   // descriptor version
    desc |= uint64_t(layout_type) << 61;
    return desc;
}

// Instruction descriptor for kind::tf32 with an FP32 accumulator: M rows
// (a multiple of 16), N columns (a multiple of 16 for M = 128); *_mn_major
// says that the operand's output index, not its reduction index, is the
// contiguous one in shared memory.
__device__ __forceinline__ uint32_t tf32_instruction(int m, int n, int a_mn_major,
                                                     int b_mn_major) {
    return (1u << 4) | (2u << 7) | (2u << 10) | (uint32_t(a_mn_major) << 15) |
           (uint32_t(b_mn_major) << 16) | (uint32_t(n >> 3) << 17) |
           (uint32_t(m >> 4) << 24);
}

}  // namespace tc
}  // namespace vitb200
