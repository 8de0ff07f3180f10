// Flash attention on the tcgen05 tensor cores (sm_100a), forward and backward,
// for long sequences and head dimensions 32 and 64.  Semantics: reference
// src/ops.c:1297-1355 (forward: P = softmax(scale Q K^T), O = P V per
// (sample, head) group, no mask) and src/ops.c:1381-1441 (backward); P is
// never stored, the forward pass keeps each row's log-sum-exp instead.
//
// All three kernels are one template.  A CTA owns a tile of 128 rows of one
// group (queries, or keys in the key/value-gradient kernel) whose operands
// stay resident in shared memory, and walks the other index in tiles of N
// columns.  For every column tile
//
//   1. "SS" products (both operands in shared memory, K-major, TF32) put a
//      128 x N block of scores into tensor memory:
//        forward            S  = Q K^T
//        query gradient     S  = Q K^T,   dP  = dO V^T
//        key/value gradient S^T = K Q^T,  dP^T = V dO^T
//   2. a group of four transform warps (one tensor-memory lane = one row per
//      thread) rewrites the block in place:
//        forward            P  = exp2(scale2 S - m)  (running maximum m, lazily
//                           raised; row sums kept in registers)
//        query gradient     dS = P o (dP - D) scale, P rebuilt from the saved
//                           log-sum-exp, D = rowsum(dO o O)
//        key/value gradient P^T and dS^T likewise, D and the log-sum-exp of the
//                           tile's queries read from a small shared table
//   3. "TS" products take that block straight from tensor memory as their A
//      operand (it never visits shared memory) and a token-major tile as B:
//        forward            O  += P V
//        query gradient     dQ += dS K
//        key/value gradient dV += P^T dO,  dK += dS^T Q
//
// Column tiles alternate between two tensor-memory buffers, each with its own
// transform group, so the tensor pipe works on tile j+1 while tile j is being
// transformed.  In the forward pass each buffer keeps its own running maximum,
// row sum and output accumulator (a split over the keys inside the CTA); the
// two halves are merged at the end.
//
// Warp roles: warp 0 issues TMA loads (3-D tensor maps [sample][token][column]
// over the token-major projection matrix or the head-major tensors, so rows
// past the end of a group read as zero and stores are clipped), warp 1 issues
// the MMAs and owns the tensor-memory allocation, warps 2-9 are the two
// transform groups and store the results (32 x 32 blocks staged in shared
// memory, TMA store or reduce-add).  Roles meet only through mbarriers; every
// wait is bounded in time, records a code in the library's status word when
// it gives up and lets the kernel run to its normal end.
#include "device_util.cuh"
#include "gemm_tc.h"
#include "kernels.h"
#include "tcgen05.cuh"

#include <algorithm>
#include <climits>
#include <cmath>
#include <cstring>
#include <unordered_map>

namespace vitb200 {
namespace {

using namespace tc;

constexpr int kTileRows = 128;
constexpr int kAttnThreads = 320;   // TMA warp, MMA warp, two groups of four
constexpr int kTmemColumns = 512;
constexpr int kBarrierBytes = 256;
constexpr int kMinSmemBytes = 116 * 1024;   // one CTA per SM: it owns all of tensor memory

constexpr int kForward = 0;
constexpr int kGradQuery = 1;
constexpr int kGradKeyValue = 2;

// kCols: columns per tile; kResident: operands that stay for the whole row
// tile; kResidentStages: buffers for them (two where shared memory allows, so
// the next item's are fetched while this item's are still in use);
// kProducts: SS products per tile; kUpdates: TS products per tile;
// kAccumulators: 128 x head_dim accumulators per work item (there are two
// sets, so that one item's results are read while the next item's grow);
// kStagingBytes: shared memory the results leave through (4 KiB per storing
// warp); kTableBytes: the transform warps' exchange table.
template <int MODE> struct Traits;
template <> struct Traits<kForward> {
    static constexpr int kCols = 128, kResident = 1, kResidentStages = 2,
                         kProducts = 1, kUpdates = 1, kAccumulators = 2,
                         kStagingBytes = 32768, kTableBytes = 2048;
};
template <> struct Traits<kGradQuery> {
    static constexpr int kCols = 96, kResident = 2, kResidentStages = 1,
                         kProducts = 2, kUpdates = 1, kAccumulators = 1,
                         kStagingBytes = 16384, kTableBytes = 0;
};
template <> struct Traits<kGradKeyValue> {
    static constexpr int kCols = 64, kResident = 2, kResidentStages = 1,
                         kProducts = 2, kUpdates = 2, kAccumulators = 2,
                         kStagingBytes = 32768, kTableBytes = 2048;
};

struct AttnMaps {
    CUtensorMap resident[2];   // 128-row boxes, K-major
    CUtensorMap ss[2];         // N-row boxes, K-major
    CUtensorMap ts[2];         // 32 x 32 boxes, 32-byte-atom swizzle
    CUtensorMap out[2];        // 32 x 32 boxes, plain FP32
};

struct AttnParams {
    int seq;
    int heads;      // groups per sample (1 when the tensors are head-major)
    int row_tiles;  // ceil(seq / 128)
    int items;      // groups * row_tiles
    float scale;    // 1 / sqrt(head_dim)
    float scale2;   // scale * log2(e)
    float *lse;               // [groups * seq]: written forward, read backward
    // [groups * seq]: D = rowsum(dO o O).  The query-gradient kernel computes
    // and writes it (from out / dout below), the key/value-gradient kernel,
    // which runs after it, reads it.
    float *row_dots;
    const float *out, *dout;  // query-gradient kernel: O and dO, for D
    int out_ld, out_heads, dout_ld, dout_heads;
    int add0, add1;           // outputs accumulate
    // Gradient kernels, optional: [gridDim.x][partial_ld] sums over the rows
    // of everything this CTA stores, output `i` at column partial_column[i] +
    // the head's offset (the bias gradient of the projection that produced Q,
    // K and V is the column sum of their gradients).  Zeroed by the caller.
    float *column_partials;
    int partial_ld;
    int partial_column[2];
    int *status;
};

enum Barrier {   // two of each
    kResidentFull = 0,
    kResidentEmpty = 2,
    kSsFull = 4,
    kSsEmpty = 6,
    kTsFull = 8,
    kTsEmpty = 10,
    kScoresFull = 12,
    kBlockReady = 14,
    kUpdateDone = 16,
    kAllDone = 18,
    kAccEmpty = 20,
    kBarriers = 22,
};

// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one() {
    uint32_t elected;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(elected));
    return elected != 0;
}

__device__ __forceinline__ void group_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Persistent: CTA c works on items c, c + gridDim.x, ... (item = one 128-row
// tile of one group; the row tiles of a group are neighbours, so CTAs that run
// side by side share the group's other operand in L2).  Column tiles are
// numbered through all of a CTA's items; tile g uses load stage, tensor-memory
// buffer and transform group g % 2, and the SS products of tile g + 2 are
// issued right after the TS products of tile g, across item boundaries, so
// the next item's first scores are computed while this item's results are
// merged and stored.
template <int HD, int MODE>
__global__ void __launch_bounds__(kAttnThreads, 1)
attention_tc_kernel(const __grid_constant__ AttnMaps maps, const AttnParams p) {
    using T = Traits<MODE>;
    constexpr int N = T::kCols;
    constexpr int kBlocks = HD / 32;   // 32-float column blocks of the head dimension
    constexpr int kResidentBytes = kTileRows * HD * 4;
    constexpr int kOperandBytes = N * HD * 4;
    constexpr int kResidentTotal = T::kResident * kResidentBytes;
    constexpr int kSsStage = T::kProducts * kOperandBytes;
    constexpr int kTsStage = T::kUpdates * kOperandBytes;
    constexpr int kBufferColumns = T::kProducts * N;
    constexpr int kAccumulatorBase = 2 * kBufferColumns;
    constexpr int kSetColumns = T::kAccumulators * HD;
    static_assert(kAccumulatorBase + 2 * kSetColumns <= kTmemColumns, "tensor memory");
    static_assert(N % 32 == 0 && HD % 32 == 0, "tile shapes");

    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t *resident = smem;
    uint8_t *ss_ring = resident + T::kResidentStages * kResidentTotal;
    uint8_t *ts_ring = ss_ring + 2 * kSsStage;
    uint8_t *staging_base = ts_ring + 2 * kTsStage;
    uint8_t *tail = staging_base + T::kStagingBytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(tail);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + kBarriers);
    volatile int *failed = reinterpret_cast<volatile int *>(tmem_slot + 1);
    float *table = reinterpret_cast<float *>(tail + kBarrierBytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int tiles = (p.seq + N - 1) / N;
    const int my_items = (p.items - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x);

    if ((smem_address(smem) & 1023u) != 0) {
        grid_dependency_wait();
        if (threadIdx.x == 0) {
            atomicExch(p.status, 16);
        }
        return;
    }
    if (threadIdx.x == 0) {
        for (int b = 0; b < kBarriers; ++b) {
            const int count = (b == kBlockReady || b == kBlockReady + 1) ? 4
                : (b == kAccEmpty || b == kAccEmpty + 1) ? 8 : 1;
            mbarrier_init(&bars[b], count);
        }
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_allocate(tmem_slot, kTmemColumns);
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base_any = *tmem_slot;
    const uint32_t tmem_base = tmem_base_any;
    // Set-up is done; everything below reads or writes global memory.
    grid_dependency_wait();
    grid_dependency_release();

    // A wait that has run out marks the CTA as failed; from then on nobody
    // waits any more and every role runs its loops to their normal end, so no
    // barrier is left with a missing participant.
    auto wait = [&](int barrier, uint32_t parity, int code) {
        if (mbarrier_try_wait(&bars[barrier], parity) || *failed) {
            return;
        }
        if (!mbarrier_wait(&bars[barrier], parity)) {
            *failed = 1;
            atomicExch(p.status, code);
        }
    };
    // Where the it-th item of this CTA lives.
    struct Item {
        int group, m0, sample, col0;
    };
    auto item_at = [&](int it) {
        const int index = int(blockIdx.x) + it * int(gridDim.x);
        Item item;
        item.group = index / p.row_tiles;
        item.m0 = (index - item.group * p.row_tiles) * kTileRows;
        item.sample = item.group / p.heads;
        item.col0 = (item.group - item.sample * p.heads) * HD;
        return item;
    };

    if (warp == 0) {
        if (lane == 0) {
            int fill = 0;   // column tiles loaded so far
            for (int it = 0; it < my_items; ++it) {
                const Item item = item_at(it);
                const int stage = it % T::kResidentStages;
                const uint32_t round = it / T::kResidentStages;
                wait(kResidentEmpty + stage, (round & 1) ^ 1, 17);
                mbarrier_expect_tx(&bars[kResidentFull + stage], kResidentTotal);
#pragma unroll
                for (int r = 0; r < T::kResident; ++r) {
#pragma unroll
                    for (int kb = 0; kb < kBlocks; ++kb) {
                        tma_load_3d(resident + stage * kResidentTotal + r * kResidentBytes +
                                        kb * (kTileRows * 128),
                                    &maps.resident[r], item.col0 + 32 * kb, item.m0,
                                    item.sample, &bars[kResidentFull + stage]);
                    }
                }
                for (int j = 0; j < tiles; ++j, ++fill) {
                    const int s = fill & 1;
                    const uint32_t phase = (fill >> 1) & 1;
                    const int n0 = j * N;
                    wait(kSsEmpty + s, phase ^ 1, 18);
                    mbarrier_expect_tx(&bars[kSsFull + s], kSsStage);
#pragma unroll
                    for (int product = 0; product < T::kProducts; ++product) {
#pragma unroll
                        for (int kb = 0; kb < kBlocks; ++kb) {
                            tma_load_3d(ss_ring + s * kSsStage + product * kOperandBytes +
                                            kb * (N * 128),
                                        &maps.ss[product], item.col0 + 32 * kb, n0,
                                        item.sample, &bars[kSsFull + s]);
                        }
                    }
                    wait(kTsEmpty + s, phase ^ 1, 19);
                    mbarrier_expect_tx(&bars[kTsFull + s], kTsStage);
#pragma unroll
                    for (int update = 0; update < T::kUpdates; ++update) {
#pragma unroll
                        for (int kk = 0; kk < N / 32; ++kk) {
#pragma unroll
                            for (int a = 0; a < kBlocks; ++a) {
                                tma_load_3d(ts_ring + s * kTsStage + update * kOperandBytes +
                                                (kk * kBlocks + a) * 4096,
                                            &maps.ts[update], item.col0 + 32 * a,
                                            n0 + 32 * kk, item.sample, &bars[kTsFull + s]);
                            }
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        {
            // One elected lane issues every MMA, but the whole warp runs the
            // control flow: values every lane computes alike live in uniform
            // registers, which is where tcgen05.mma takes its operands from
            // (inside a one-lane branch each operand would be moved there
            // instruction by instruction).  The descriptors are built once
            // (high word constant, low word = address field + leading offset)
            // and stepped by adding compile-time constants to the low word.
            const uint32_t leader = elect_one() ? 1u : 0u;
            const uint32_t tmem_base = __shfl_sync(kFullMask, tmem_base_any, 0);
            const uint32_t update_instruction = tf32_instruction(kTileRows, HD, 0, 1);
            const uint32_t full_instruction = tf32_instruction(kTileRows, N, 0, 0);
            // K-major: 8-row groups 1024 bytes apart (stride), K steps of 32
            // bytes inside the 128-byte swizzled row, one 32-float block of
            // the head dimension after the other.
            constexpr uint32_t kHighKMajor = (1024u >> 4) | (1u << 14) |
                                             (kLayoutSwizzle128 << 29);
            // Output index contiguous, 32-byte-atom swizzle: boxes of one
            // 32-row reduction block 4096 bytes apart (leading offset),
            // groups of four rows 512 bytes apart, K steps of eight rows.
            constexpr uint32_t kHighBox32 = (512u >> 4) | (1u << 14) |
                                            (kLayoutSwizzle128Base32 << 29);
            auto descriptor = [](uint32_t low, uint32_t high) {
                return (uint64_t(high) << 32) | low;
            };
            auto low_word = [](uint32_t address, uint32_t leading_bytes) {
                return ((address >> 4) & 0x3fffu) | ((leading_bytes >> 4) << 16);
            };
            const uint32_t resident_low = low_word(smem_address(resident), 16);
            const uint32_t ss_low = low_word(smem_address(ss_ring), 16);
            const uint32_t ts_low = low_word(smem_address(ts_ring), 4096);
            const int total = my_items * tiles;
            // SS products of column tile g into buffer g % 2.
            int scores_it = 0, scores_j = 0;
            auto scores = [&](int g) {
                const int s = g & 1;
                const int stage = scores_it % T::kResidentStages;
                if (scores_j == 0) {
                    wait(kResidentFull + stage, (scores_it / T::kResidentStages) & 1, 20);
                }
                wait(kSsFull + s, (g >> 1) & 1, 21);
                tcgen05_fence_after();
                const int valid = p.seq - scores_j * N;
                const uint32_t instruction = valid >= N
                    ? full_instruction
                    : tf32_instruction(kTileRows, (valid + 15) & ~15, 0, 0);
#pragma unroll
                for (int product = 0; product < T::kProducts; ++product) {
                    const uint32_t d = tmem_base + s * kBufferColumns + product * N;
                    const uint32_t a_low =
                        resident_low + ((stage * kResidentTotal + product * kResidentBytes) >> 4);
                    const uint32_t b_low =
                        ss_low + ((s * kSsStage + product * kOperandBytes) >> 4);
#pragma unroll
                    for (int ks = 0; ks < HD / 8; ++ks) {
                        constexpr int kRowBlock = kTileRows * 128, kColBlock = N * 128;
                        tcgen05_mma_tf32_if(
                            leader, d,
                            descriptor(a_low + (((ks / 4) * kRowBlock + (ks % 4) * 32) >> 4),
                                       kHighKMajor),
                            descriptor(b_low + (((ks / 4) * kColBlock + (ks % 4) * 32) >> 4),
                                       kHighKMajor),
                            instruction, ks > 0 ? 1u : 0u);
                    }
                }
                tcgen05_commit_if(leader, &bars[kSsEmpty + s]);
                tcgen05_commit_if(leader, &bars[kScoresFull + s]);
                if (++scores_j == tiles) {
                    // The item's resident operands have been read for the
                    // last time once these products retire.
                    tcgen05_commit_if(leader, &bars[kResidentEmpty + stage]);
                    scores_j = 0;
                    ++scores_it;
                }
            };
            // TS products of column tile g: A = the transformed block in
            // tensor memory (eight columns per K step), B = 32 x 32 boxes.
            int update_it = 0, update_j = 0;
            auto update = [&](int g) {
                const int s = g & 1;
                const uint32_t phase = (g >> 1) & 1;
                const int set = update_it & 1;
                wait(kBlockReady + s, phase, 22);
                wait(kTsFull + s, phase, 23);
                if (update_j == 0) {
                    // The transform warps must have read this accumulator
                    // set's previous contents (two items ago).
                    wait(kAccEmpty + set, ((update_it >> 1) & 1) ^ 1, 24);
                }
                tcgen05_fence_after();
                const int valid = min(N, p.seq - update_j * N);
                const int steps = (valid + 7) >> 3;
#pragma unroll
                for (int u = 0; u < T::kUpdates; ++u) {
                    const int accumulator = MODE == kForward ? s : u;
                    const bool first = MODE == kForward ? update_j < 2 : update_j == 0;
                    const uint32_t d = tmem_base + kAccumulatorBase + set * kSetColumns +
                                       accumulator * HD;
                    const uint32_t a = tmem_base + s * kBufferColumns + u * N;
                    const uint32_t b_low = ts_low + ((s * kTsStage + u * kOperandBytes) >> 4);
                    tcgen05_mma_tf32_tmem_a_if(leader, d, a, descriptor(b_low, kHighBox32),
                                               update_instruction, first ? 0u : 1u);
#pragma unroll
                    for (int ks = 1; ks < N / 8; ++ks) {
                        if (ks < steps) {
                            tcgen05_mma_tf32_tmem_a_if(
                                leader, d, a + 8 * ks,
                                descriptor(b_low + (((ks / 4) * (kBlocks * 4096) +
                                                     (ks % 4) * 1024) >> 4),
                                           kHighBox32),
                                update_instruction, 1u);
                        }
                    }
                }
                tcgen05_commit_if(leader, &bars[kTsEmpty + s]);
                tcgen05_commit_if(leader, &bars[kUpdateDone + s]);
                if (++update_j == tiles) {
                    tcgen05_commit_if(leader, &bars[kAllDone + set]);
                    update_j = 0;
                    ++update_it;
                }
            };
            if (total > 0) {
                scores(0);
            }
            if (total > 1) {
                scores(1);
            }
            for (int g = 0; g < total; ++g) {
                update(g);
                if (g + 2 < total) {
                    scores(g + 2);
                }
            }
        }
    } else {
        const int wg = (warp - 2) >> 2;       // transform group = buffer
        const int quarter = warp & 3;         // tensor-memory lanes this warp may touch
        const int row = quarter * 32 + lane;  // row of the tile this thread owns
        const uint32_t lane_base = tmem_base + (uint32_t(quarter * 32) << 16);
        const uint32_t block_address = lane_base + wg * kBufferColumns;
        float *staging = reinterpret_cast<float *>(
            staging_base + ((T::kStagingBytes == 32768 ? wg * 4 : 0) + quarter) * 4096);
        bool staged = false;   // this warp has a store in flight from `staging`
        int visit = 0;         // column tiles this group has transformed so far

        // Stages r[] (this lane's 32 values of a 32 x 32 block) in the
        // 128-byte swizzle the store map expects and hands it to the copy
        // engine.  Rows past the end of the group are clipped by the map.
        auto store_block = [&](uint32_t (&r)[32], const CUtensorMap *map, const Item &item,
                               int column, bool add, int partial_column) {
            if (staged) {
                if (lane == 0) {
                    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                }
                __syncwarp();
            }
            staged = true;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                float4 v;
                v.x = __uint_as_float(r[4 * c + 0]);
                v.y = __uint_as_float(r[4 * c + 1]);
                v.z = __uint_as_float(r[4 * c + 2]);
                v.w = __uint_as_float(r[4 * c + 3]);
                *reinterpret_cast<float4 *>(staging + lane * 32 + 4 * (c ^ (lane & 7))) = v;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0 && item.m0 + quarter * 32 < p.seq) {
                if (add) {
                    tma_reduce_add_3d(staging, map, item.col0 + column,
                                      item.m0 + quarter * 32, item.sample);
                } else {
                    tma_store_3d(staging, map, item.col0 + column,
                                 item.m0 + quarter * 32, item.sample);
                }
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
            if (MODE != kForward && p.column_partials) {
                // Column sums of the block's live rows, lane = column (the
                // swizzle keeps a row's 32 words in 32 different banks), read
                // while the copy engine reads the block too.
                const int live = min(32, p.seq - (item.m0 + quarter * 32));
                float sum = 0.0f;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    if (i < live) {
                        sum += staging[i * 32 + 4 * ((lane >> 2) ^ (i & 7)) + (lane & 3)];
                    }
                }
                if (live > 0) {
                    atomicAdd(p.column_partials + size_t(blockIdx.x) * p.partial_ld +
                                  partial_column + item.col0 + column + lane,
                              sum);
                }
            }
        };
        auto publish_block = [&]() {
            tcgen05_wait_store();
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbarrier_arrive(&bars[kBlockReady + wg]);
            }
        };
        // The accumulators of item `it` are complete / have been read.
        auto await_results = [&](int it) {
            wait(kAllDone + (it & 1), (it >> 1) & 1, 27);
            tcgen05_fence_after();
        };
        auto release_results = [&](int it) {
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbarrier_arrive(&bars[kAccEmpty + (it & 1)]);
            }
        };

        // The tensor cores drop the low 13 mantissa bits of an FP32 word in
        // tensor memory.  Values written there are scaled by 1 + 2^-11 first
        // (folded into an exponent or a factor that is applied anyway), which
        // turns that truncation into rounding to nearest on average at no
        // cost per element.
        constexpr float kRoundUp = 1.00048828125f;            // 1 + 2^-11
        constexpr float kRoundUpLog2 = 0.000704269011247f;    // log2(1 + 2^-11)

        // Results of item `it` are merged / stored one tile into item it + 1
        // (see the loops below): by then the next scores this group needs
        // have been turned into work for the tensor pipe, so the stores and
        // the wait for the item's last products stay off the critical path.
        if constexpr (MODE == kForward) {
            float reference = -INFINITY;   // running maximum, in units of scale2 * score
            float sum = 0.0f;              // row sum of P (times 1 + 2^-11)
            float done_reference = 0.0f, done_sum = 0.0f;   // of the item awaiting its merge
            // Merge the two groups' halves: O = (w0 O0 + w1 O1) / (w0 l0 +
            // w1 l1) with w = 2^(m - max(m0, m1)); a group that saw no tile
            // has l = 0 and its accumulator is not read.
            auto finish = [&](int it) {
                const Item item = item_at(it);
                const int first_tile = it * tiles;
                const uint32_t set_address =
                    lane_base + kAccumulatorBase + (it & 1) * kSetColumns;
                float *stats = table;
                stats[wg * kTileRows + row] = done_reference;
                stats[256 + wg * kTileRows + row] = done_sum;
                group_barrier(1, 256);
                const float m_a = stats[row], m_b = stats[kTileRows + row];
                const float l_a = stats[256 + row], l_b = stats[256 + kTileRows + row];
                group_barrier(1, 256);   // the table may be rewritten from here on
                const float top = fmaxf(m_a, m_b);
                const float w_a = l_a > 0.0f ? exp2_approx(m_a - top) : 0.0f;
                const float w_b = l_b > 0.0f ? exp2_approx(m_b - top) : 0.0f;
                const float total = l_a * w_a + l_b * w_b;
                const float inverse = kRoundUp / total;
                if (wg == 0 && p.lse && item.m0 + row < p.seq) {
                    p.lse[size_t(item.group) * p.seq + item.m0 + row] =
                        top + log2f(total) - kRoundUpLog2;
                }
                const bool use_a = tiles > 1 || (first_tile & 1) == 0;
                const bool use_b = tiles > 1 || (first_tile & 1) == 1;
                await_results(it);
                uint32_t r[32];
                const int block = wg;   // group 0: columns 0..31, group 1: 32..63
                if (block < kBlocks) {
                    uint32_t other[32];
                    if (use_a) {
                        tcgen05_load_32(set_address + 32 * block, r);
                    }
                    if (use_b) {
                        tcgen05_load_32(set_address + HD + 32 * block, other);
                    }
#pragma unroll
                    for (int e = 0; e < 32; ++e) {
                        const float a = use_a ? __uint_as_float(r[e]) * w_a : 0.0f;
                        const float b = use_b ? __uint_as_float(other[e]) * w_b : 0.0f;
                        r[e] = __float_as_uint((a + b) * inverse);
                    }
                }
                release_results(it);
                if (block < kBlocks) {
                    store_block(r, &maps.out[0], item, 32 * block, false, 0);
                }
            };
            // One loop body for "transform the group's next tile" and "finish
            // the previous item" (after the first tile of the next item, or
            // at once when this group has no tile there).
            int it = 0, j = wg;
            bool seen = false, owed = false;
            while (it < my_items || owed) {
                const bool tile = it < my_items && j < tiles;
                if (tile) {
                    // Online softmax over this group's share of the key
                    // tiles.  The reference maximum is raised only when a tile
                    // exceeds it by more than 2^8, so the output accumulator
                    // is rescaled rarely.
                    const uint32_t output =
                        lane_base + kAccumulatorBase + (it & 1) * kSetColumns + wg * HD;
                    wait(kScoresFull + wg, visit & 1, 25);
                    tcgen05_fence_after();
                    const int valid = min(N, p.seq - j * N);
                    // Columns are handled 64 at a time (32 in the ragged last
                    // block), once for the maximum and once for the
                    // exponentials; columns past the end of the group count
                    // as -inf / 0.
                    float top[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
                    if (valid == N) {
#pragma unroll 1
                        for (int half = 0; half < 2; ++half) {
                            uint32_t r[64];
                            tcgen05_load_64(block_address + 64 * half, r);
#pragma unroll
                            for (int e = 0; e < 64; ++e) {
                                top[e & 3] = fmaxf(top[e & 3], __uint_as_float(r[e]));
                            }
                        }
                    } else {
#pragma unroll 1
                        for (int c = 0; 32 * c < valid; ++c) {
                            uint32_t r[32];
                            tcgen05_load_32(block_address + 32 * c, r);
                            const int live = valid - 32 * c;
#pragma unroll
                            for (int e = 0; e < 32; ++e) {
                                if (e < live) {
                                    top[e & 3] = fmaxf(top[e & 3], __uint_as_float(r[e]));
                                }
                            }
                        }
                    }
                    const float tile_max =
                        fmaxf(fmaxf(top[0], top[1]), fmaxf(top[2], top[3])) * p.scale2;
                    const bool raise = tile_max > reference + 8.0f;
                    float factor = 1.0f;
                    if (raise) {
                        factor = exp2_approx(reference - tile_max);   // 0 the first time
                        reference = tile_max;
                        sum *= factor;
                    }
                    if (seen && __any_sync(kFullMask, raise)) {
                        wait(kUpdateDone + wg, (visit - 1) & 1, 26);
                        tcgen05_fence_after();
#pragma unroll
                        for (int c = 0; c < kBlocks; ++c) {
                            uint32_t o[32];
                            tcgen05_load_32(output + 32 * c, o);
#pragma unroll
                            for (int e = 0; e < 32; ++e) {
                                o[e] = __float_as_uint(__uint_as_float(o[e]) * factor);
                            }
                            tcgen05_store_32(output + 32 * c, o);
                        }
                    }
                    const float shift = kRoundUpLog2 - reference;
                    float part[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    if (valid == N) {
#pragma unroll 1
                        for (int half = 0; half < 2; ++half) {
                            uint32_t r[64];
                            tcgen05_load_64(block_address + 64 * half, r);
#pragma unroll
                            for (int e = 0; e < 64; ++e) {
                                const float value =
                                    exp2_approx(fmaf(__uint_as_float(r[e]), p.scale2, shift));
                                part[e & 3] += value;
                                r[e] = __float_as_uint(value);
                            }
                            tcgen05_store_64(block_address + 64 * half, r);
                        }
                    } else {
#pragma unroll 1
                        for (int c = 0; 32 * c < valid; ++c) {
                            uint32_t r[32];
                            tcgen05_load_32(block_address + 32 * c, r);
                            const int live = valid - 32 * c;
#pragma unroll
                            for (int e = 0; e < 32; ++e) {
                                float value =
                                    exp2_approx(fmaf(__uint_as_float(r[e]), p.scale2, shift));
                                if (e >= live) {
                                    value = 0.0f;
                                }
                                part[e & 3] += value;
                                r[e] = __float_as_uint(value);
                            }
                            tcgen05_store_32(block_address + 32 * c, r);
                        }
                    }
                    sum += (part[0] + part[1]) + (part[2] + part[3]);
                    publish_block();
                    seen = true;
                    j += 2;
                    ++visit;
                }
                if (owed) {
                    finish(it - 1);
                    owed = false;
                }
                if (!tile) {
                    if (it >= my_items) {
                        break;
                    }
                    done_reference = reference;
                    done_sum = sum;
                    reference = -INFINITY;
                    sum = 0.0f;
                    seen = false;
                    ++it;
                    j = ((it * tiles) & 1) ^ wg;
                    owed = true;
                }
            }
        } else if constexpr (MODE == kGradQuery) {
            auto finish = [&](int it) {
                const Item item = item_at(it);
                await_results(it);
                if (wg == 0) {
                    // One group stores; the other goes on with its tiles.
                    const uint32_t set_address =
                        lane_base + kAccumulatorBase + (it & 1) * kSetColumns;
                    uint32_t r[kBlocks][32];
#pragma unroll
                    for (int block = 0; block < kBlocks; ++block) {
                        tcgen05_load_32(set_address + 32 * block, r[block]);
                    }
                    release_results(it);
#pragma unroll
                    for (int block = 0; block < kBlocks; ++block) {
                        store_block(r[block], &maps.out[0], item, 32 * block, p.add0 != 0,
                                    p.partial_column[0]);
                    }
                } else {
                    release_results(it);
                }
            };
            const float factor = p.scale * kRoundUp;
            int it = 0, j = wg;
            bool owed = false, fresh = true;
            float row_lse = 0.0f, row_dot = 0.0f;
            while (it < my_items || owed) {
                const bool tile = it < my_items && j < tiles;
                if (tile) {
                    if (fresh) {
                        // This row's log-sum-exp and D = dO . O (both groups
                        // compute it, one writes it for the kernel that
                        // follows).  The loads are in flight while the
                        // item's first scores are being computed.
                        const Item item = item_at(it);
                        const int q = item.m0 + row;
                        row_lse = 0.0f;
                        row_dot = 0.0f;
                        if (q < p.seq && HD > 32) {
                            // Wide heads: D was computed by the kernel before
                            // this one (a row here is 256 bytes per operand;
                            // fetching it per thread costs more than it saves).
                            const size_t at = size_t(item.group) * p.seq + q;
                            row_lse = p.lse[at];
                            row_dot = p.row_dots[at];
                        } else if (q < p.seq) {
                            const size_t at = size_t(item.group) * p.seq + q;
                            row_lse = p.lse[at];
                            const float4 *o = reinterpret_cast<const float4 *>(
                                p.out +
                                (size_t(item.group / p.out_heads) * p.seq + q) * p.out_ld +
                                size_t(item.group % p.out_heads) * HD);
                            const float4 *g = reinterpret_cast<const float4 *>(
                                p.dout +
                                (size_t(item.group / p.dout_heads) * p.seq + q) * p.dout_ld +
                                size_t(item.group % p.dout_heads) * HD);
                            float part[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                            for (int i = 0; i < HD / 4; ++i) {
                                const float4 x = __ldg(o + i), y = __ldg(g + i);
                                part[i & 3] += x.x * y.x + x.y * y.y + x.z * y.z + x.w * y.w;
                            }
                            row_dot = (part[0] + part[1]) + (part[2] + part[3]);
                            if (wg == 0) {
                                p.row_dots[at] = row_dot;
                            }
                        }
                        fresh = false;
                    }
                    wait(kScoresFull + wg, visit & 1, 25);
                    tcgen05_fence_after();
                    const int valid = min(N, p.seq - j * N);
                    const int chunks = (valid + 31) >> 5;
#pragma unroll 1
                    for (int c = 0; c < chunks; ++c) {
                        uint32_t s[32], g[32];
                        tcgen05_load_32_pair(block_address + 32 * c,
                                             block_address + N + 32 * c, s, g);
#pragma unroll
                        for (int e = 0; e < 32; ++e) {
                            const float probability = exp2_approx(
                                fmaf(__uint_as_float(s[e]), p.scale2, -row_lse));
                            s[e] = __float_as_uint(
                                probability * ((__uint_as_float(g[e]) - row_dot) * factor));
                        }
                        tcgen05_store_32(block_address + 32 * c, s);
                    }
                    publish_block();
                    j += 2;
                    ++visit;
                }
                if (owed) {
                    finish(it - 1);
                    owed = false;
                }
                if (!tile) {
                    if (it >= my_items) {
                        break;
                    }
                    ++it;
                    j = ((it * tiles) & 1) ^ wg;
                    owed = true;
                    fresh = true;
                }
            }
        } else {
            static_assert(MODE != kGradKeyValue || N == 64, "table size");
            // Rows are keys, columns the queries of tile j: their log-sum-exp
            // (less log2(1 + 2^-11)) and D come from a table in shared
            // memory, fetched one visit ahead by this group's 128 threads (64
            // of each).
            float2 *pairs = reinterpret_cast<float2 *>(table) + wg * 2 * N;
            const int t = int(threadIdx.x) - 64 - wg * 128;
            // The tile this group transforms after (it, j); false at the end.
            auto advance = [&](int &it, int &j) {
                j += 2;
                while (j >= tiles) {
                    if (++it >= my_items) {
                        return false;
                    }
                    j = ((it * tiles) & 1) ^ wg;
                }
                return true;
            };
            auto fetch = [&](int it, int j) {
                const Item item = item_at(it);
                const int q = j * N + (t & (N - 1));
                if (q >= p.seq) {
                    return 0.0f;
                }
                const size_t at = size_t(item.group) * p.seq + q;
                return t < N ? p.lse[at] - kRoundUpLog2 : p.row_dots[at];
            };
            auto put = [&](int buffer, float value) {
                float *pair = reinterpret_cast<float *>(pairs + buffer * N + (t & (N - 1)));
                pair[t < N ? 0 : 1] = value;
            };
            // Group 0 stores dV, group 1 stores dK.
            auto finish = [&](int it) {
                const Item item = item_at(it);
                await_results(it);
                const uint32_t mine =
                    lane_base + kAccumulatorBase + (it & 1) * kSetColumns + wg * HD;
                uint32_t r[kBlocks][32];
#pragma unroll
                for (int block = 0; block < kBlocks; ++block) {
                    tcgen05_load_32(mine + 32 * block, r[block]);
                }
                release_results(it);
#pragma unroll
                for (int block = 0; block < kBlocks; ++block) {
                    store_block(r[block], &maps.out[wg], item, 32 * block,
                                (wg ? p.add1 : p.add0) != 0,
                                wg ? p.partial_column[1] : p.partial_column[0]);
                }
            };
            int ahead_it = 0, ahead_j = wg - 2;
            bool ahead = my_items > 0 && advance(ahead_it, ahead_j);
            if (ahead) {
                put(0, fetch(ahead_it, ahead_j));
                ahead = advance(ahead_it, ahead_j);
            }
            int it = 0, j = wg;
            bool owed = false;
            while (it < my_items || owed) {
                const bool tile = it < my_items && j < tiles;
                if (tile) {
                    const float next = ahead ? fetch(ahead_it, ahead_j) : 0.0f;
                    group_barrier(2 + wg, 128);
                    wait(kScoresFull + wg, visit & 1, 25);
                    tcgen05_fence_after();
                    const float2 *columns = pairs + (visit & 1) * N;
                    const int valid = min(N, p.seq - j * N);
                    const int chunks = (valid + 31) >> 5;
#pragma unroll 1
                    for (int c = 0; c < chunks; ++c) {
                        uint32_t s[32], g[32];
                        tcgen05_load_32_pair(block_address + 32 * c,
                                             block_address + N + 32 * c, s, g);
#pragma unroll
                        for (int e = 0; e < 32; e += 2) {
                            const float4 two =
                                *reinterpret_cast<const float4 *>(columns + 32 * c + e);
                            const float p0 = exp2_approx(
                                fmaf(__uint_as_float(s[e]), p.scale2, -two.x));
                            const float p1 = exp2_approx(
                                fmaf(__uint_as_float(s[e + 1]), p.scale2, -two.z));
                            g[e] = __float_as_uint(
                                p0 * ((__uint_as_float(g[e]) - two.y) * p.scale));
                            g[e + 1] = __float_as_uint(
                                p1 * ((__uint_as_float(g[e + 1]) - two.w) * p.scale));
                            s[e] = __float_as_uint(p0);
                            s[e + 1] = __float_as_uint(p1);
                        }
                        tcgen05_store_32(block_address + 32 * c, s);
                        tcgen05_store_32(block_address + N + 32 * c, g);
                    }
                    publish_block();
                    if (ahead) {
                        put((visit + 1) & 1, next);
                        ahead = advance(ahead_it, ahead_j);
                    }
                    j += 2;
                    ++visit;
                }
                if (owed) {
                    finish(it - 1);
                    owed = false;
                }
                if (!tile) {
                    if (it >= my_items) {
                        break;
                    }
                    ++it;
                    j = ((it * tiles) & 1) ^ wg;
                    owed = true;
                }
            }
        }
        if (lane == 0) {
            asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tcgen05_fence_after();
        tmem_free(tmem_base, kTmemColumns);
    }
}

// dots[g * seq + t] = sum_c dO[g, t, c] * O[g, t, c] for 64-wide heads: sixteen
// lanes per row (one float4 of each operand per lane: 256 contiguous bytes per
// row), two rows per warp and load, four such pairs in flight.
__global__ void __launch_bounds__(256)
attention_row_dots_kernel(const float *__restrict__ out, const float *__restrict__ dout,
                          float *__restrict__ dots, size_t rows, int seq,
                          HeadLayout out_layout, HeadLayout dout_layout) {
    constexpr int HD = 64;
    grid_dependency_wait();
    grid_dependency_release();
    const int lane = threadIdx.x & 31;
    const int part = lane & 15;
    const size_t warps = grid_threads() >> 5;
    for (size_t first = (global_thread() >> 5) * 8; first < rows; first += warps * 8) {
        float sums[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const size_t r = first + 2 * i + (lane >> 4);
            sums[i] = 0.0f;
            if (r < rows) {
                const size_t group = r / size_t(seq), t = r % size_t(seq);
                const float4 x = __ldg(reinterpret_cast<const float4 *>(
                    out + ((group / out_layout.heads) * seq + t) * size_t(out_layout.ld) +
                    (group % out_layout.heads) * HD) + part);
                const float4 y = __ldg(reinterpret_cast<const float4 *>(
                    dout + ((group / dout_layout.heads) * seq + t) * size_t(dout_layout.ld) +
                    (group % dout_layout.heads) * HD) + part);
                sums[i] = x.x * y.x + x.y * y.y + x.z * y.z + x.w * y.w;
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
#pragma unroll
            for (int offset = 8; offset > 0; offset >>= 1) {
                sums[i] += __shfl_xor_sync(kFullMask, sums[i], offset);
            }
            const size_t r = first + 2 * i + (lane >> 4);
            if (part == 0 && r < rows) {
                dots[r] = sums[i];
            }
        }
    }
}

// ---- host side -------------------------------------------------------------

using EncodeTiled = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t,
                                 void *, const cuuint64_t *, const cuuint64_t *,
                                 const cuuint32_t *, const cuuint32_t *,
                                 CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
    static EncodeTiled function = []() -> EncodeTiled {
        void *entry = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry,
                                    cudaEnableDefault, &result) != cudaSuccess ||
            result != cudaDriverEntryPointSuccess) {
            return nullptr;
        }
        return reinterpret_cast<EncodeTiled>(entry);
    }();
    return function;
}

struct MapKey {
    const void *base;
    int ld, heads, seq, samples, head_dim, box_rows, kind;
    bool operator==(const MapKey &o) const {
        return base == o.base && ld == o.ld && heads == o.heads && seq == o.seq &&
               samples == o.samples && head_dim == o.head_dim &&
               box_rows == o.box_rows && kind == o.kind;
    }
};

struct MapKeyHash {
    size_t operator()(const MapKey &k) const {
        size_t h = reinterpret_cast<size_t>(k.base);
        for (int v : {k.ld, k.heads, k.seq, k.samples, k.head_dim, k.box_rows, k.kind}) {
            h = h * 1000003u ^ size_t(v);
        }
        return h;
    }
};

constexpr int kMapKMajor = 0;   // TF32, 128-byte swizzle, 32 x box_rows
constexpr int kMapBox32 = 1;    // TF32, 32-byte-atom swizzle, 32 x 32
constexpr int kMapStore = 2;    // FP32, 128-byte swizzle, 32 x 32

// [samples][seq][heads * head_dim] view of a tensor whose rows are `ld` floats
// apart: the token-major projection matrix (heads > 1, base = first column of
// Q, K or V) or a head-major tensor (heads = 1, ld = head_dim, one "sample"
// per group).  Rows past `seq` read as zero and are not written.
bool group_map(const float *base, HeadLayout layout, size_t groups, size_t seq,
               int head_dim, int box_rows, int kind, CUtensorMap *out) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    const int samples = int(groups / size_t(layout.heads));
    const MapKey key{base, layout.ld, layout.heads, int(seq), samples, head_dim,
                     box_rows, kind};
    auto found = cache.find(key);
    if (found != cache.end()) {
        *out = found->second;
        return true;
    }
    EncodeTiled encode = encode_tiled();
    if (!encode) {
        return false;
    }
    const cuuint64_t dims[3] = {cuuint64_t(layout.heads) * head_dim, seq,
                                cuuint64_t(samples)};
    const cuuint64_t strides[2] = {cuuint64_t(layout.ld) * sizeof(float),
                                   cuuint64_t(seq) * layout.ld * sizeof(float)};
    const cuuint32_t box[3] = {32, cuuint32_t(box_rows), 1};
    const cuuint32_t element_strides[3] = {1, 1, 1};
    const CUresult status = encode(
        out,
        kind == kMapStore ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                          : CU_TENSOR_MAP_DATA_TYPE_TFLOAT32,
        3, const_cast<float *>(base), dims, strides, box, element_strides,
        CU_TENSOR_MAP_INTERLEAVE_NONE,
        kind == kMapBox32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                          : CU_TENSOR_MAP_SWIZZLE_128B,
        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (status != CUDA_SUCCESS) {
        return false;
    }
    if (cache.size() > 4096) {
        cache.clear();
    }
    cache.emplace(key, *out);
    return true;
}

HeadLayout resolved(HeadLayout layout, size_t head_dim) {
    if (layout.ld == 0) {
        layout.ld = int(head_dim);
        layout.heads = 1;
    }
    return layout;
}

bool operand_ok(const void *pointer, HeadLayout layout, size_t groups) {
    return (reinterpret_cast<uintptr_t>(pointer) & 15) == 0 && layout.ld % 4 == 0 &&
           layout.heads >= 1 && groups % size_t(layout.heads) == 0;
}

template <int HD, int MODE>
constexpr int smem_bytes() {
    using T = Traits<MODE>;
    const int bytes = T::kResidentStages * T::kResident * kTileRows * HD * 4 +
                      2 * (T::kProducts + T::kUpdates) * T::kCols * HD * 4 +
                      T::kStagingBytes + kBarrierBytes + T::kTableBytes;
    return bytes < kMinSmemBytes ? kMinSmemBytes : bytes;
}

template <int HD, int MODE>
bool launch(const AttnMaps &maps, AttnParams params, size_t groups,
            cudaStream_t stream) {
    static bool configured = false;
    constexpr int bytes = smem_bytes<HD, MODE>();
    static_assert(bytes <= 227 * 1024, "shared memory");
    if (!configured) {
        if (cudaFuncSetAttribute(attention_tc_kernel<HD, MODE>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 bytes) != cudaSuccess) {
            return false;
        }
        configured = true;
    }
    const size_t items = groups * size_t(params.row_tiles);
    if (items > size_t(INT_MAX)) {
        return false;
    }
    params.items = int(items);
    // One persistent CTA per SM (it owns the SM's tensor memory).
    const unsigned grid = unsigned(std::min<size_t>(items, size_t(device_sm_count())));
    launch_chained(attention_tc_kernel<HD, MODE>, grid, kAttnThreads, bytes,
                   stream, maps, params);
    ++g_kernel_launches;
    return true;
}

AttnParams base_params(size_t seq, int heads, float scale) {
    AttnParams params;
    memset(&params, 0, sizeof(params));
    params.seq = int(seq);
    params.heads = heads;
    params.row_tiles = int((seq + kTileRows - 1) / kTileRows);
    params.scale = scale;
    params.scale2 = scale * 1.4426950408889634f;
    params.status = tc_status_device_pointer();
    return params;
}

}  // namespace

bool attention_tc_supported(size_t seq, size_t head_dim) {
    return (head_dim == 32 || head_dim == 64) && seq >= 1 && seq <= (1u << 20);
}

bool launch_attention_tc_forward(const float *q, const float *k, const float *v,
                                 float *out, float *lse, size_t groups, size_t seq,
                                 size_t head_dim, float scale, cudaStream_t stream,
                                 HeadLayout in_layout, HeadLayout out_layout) {
    if (!attention_tc_supported(seq, head_dim) || groups == 0) {
        return false;
    }
    in_layout = resolved(in_layout, head_dim);
    out_layout = resolved(out_layout, head_dim);
    if (!operand_ok(q, in_layout, groups) || !operand_ok(k, in_layout, groups) ||
        !operand_ok(v, in_layout, groups) || !operand_ok(out, out_layout, groups)) {
        return false;
    }
    const int hd = int(head_dim);
    AttnMaps maps;
    memset(&maps, 0, sizeof(maps));
    constexpr int N = Traits<kForward>::kCols;
    if (!group_map(q, in_layout, groups, seq, hd, kTileRows, kMapKMajor, &maps.resident[0]) ||
        !group_map(k, in_layout, groups, seq, hd, N, kMapKMajor, &maps.ss[0]) ||
        !group_map(v, in_layout, groups, seq, hd, 32, kMapBox32, &maps.ts[0]) ||
        !group_map(out, out_layout, groups, seq, hd, 32, kMapStore, &maps.out[0])) {
        return false;
    }
    AttnParams params = base_params(seq, in_layout.heads, scale);
    if (!params.status || out_layout.heads != in_layout.heads) {
        return false;
    }
    params.lse = lse;
    return hd == 32 ? launch<32, kForward>(maps, params, groups, stream)
                    : launch<64, kForward>(maps, params, groups, stream);
}

size_t attention_tc_partial_rows() {
    return device_sm_count();
}

bool launch_attention_tc_backward(const float *q, const float *k, const float *v,
                                  const float *out, const float *dout,
                                  const float *lse, float *dq, float *dk, float *dv,
                                  float *row_dots, size_t groups, size_t seq,
                                  size_t head_dim, float scale, bool add_q,
                                  bool add_k, bool add_v, cudaStream_t stream,
                                  HeadLayout in_layout, HeadLayout out_layout,
                                  HeadLayout dout_layout, HeadLayout grad_layout,
                                  float *column_partials) {
    if (!attention_tc_supported(seq, head_dim) || groups == 0) {
        return false;
    }
    if (column_partials && (add_q || add_k || add_v)) {
        return false;   // the sums would lack what the outputs already hold
    }
    in_layout = resolved(in_layout, head_dim);
    out_layout = resolved(out_layout, head_dim);
    dout_layout = resolved(dout_layout, head_dim);
    grad_layout = resolved(grad_layout, head_dim);
    if (!operand_ok(q, in_layout, groups) || !operand_ok(k, in_layout, groups) ||
        !operand_ok(v, in_layout, groups) || !operand_ok(dout, dout_layout, groups) ||
        !operand_ok(dq, grad_layout, groups) || !operand_ok(dk, grad_layout, groups) ||
        !operand_ok(dv, grad_layout, groups) || !operand_ok(out, out_layout, groups) ||
        (reinterpret_cast<uintptr_t>(row_dots) & 3) != 0 ||
        in_layout.heads != dout_layout.heads || in_layout.heads != grad_layout.heads) {
        return false;
    }
    const int hd = int(head_dim);
    AttnMaps query_maps, key_maps;
    memset(&query_maps, 0, sizeof(query_maps));
    memset(&key_maps, 0, sizeof(key_maps));
    constexpr int NQ = Traits<kGradQuery>::kCols;
    constexpr int NK = Traits<kGradKeyValue>::kCols;
    if (!group_map(q, in_layout, groups, seq, hd, kTileRows, kMapKMajor, &query_maps.resident[0]) ||
        !group_map(dout, dout_layout, groups, seq, hd, kTileRows, kMapKMajor, &query_maps.resident[1]) ||
        !group_map(k, in_layout, groups, seq, hd, NQ, kMapKMajor, &query_maps.ss[0]) ||
        !group_map(v, in_layout, groups, seq, hd, NQ, kMapKMajor, &query_maps.ss[1]) ||
        !group_map(k, in_layout, groups, seq, hd, 32, kMapBox32, &query_maps.ts[0]) ||
        !group_map(dq, grad_layout, groups, seq, hd, 32, kMapStore, &query_maps.out[0]) ||
        !group_map(k, in_layout, groups, seq, hd, kTileRows, kMapKMajor, &key_maps.resident[0]) ||
        !group_map(v, in_layout, groups, seq, hd, kTileRows, kMapKMajor, &key_maps.resident[1]) ||
        !group_map(q, in_layout, groups, seq, hd, NK, kMapKMajor, &key_maps.ss[0]) ||
        !group_map(dout, dout_layout, groups, seq, hd, NK, kMapKMajor, &key_maps.ss[1]) ||
        !group_map(dout, dout_layout, groups, seq, hd, 32, kMapBox32, &key_maps.ts[0]) ||
        !group_map(q, in_layout, groups, seq, hd, 32, kMapBox32, &key_maps.ts[1]) ||
        !group_map(dv, grad_layout, groups, seq, hd, 32, kMapStore, &key_maps.out[0]) ||
        !group_map(dk, grad_layout, groups, seq, hd, 32, kMapStore, &key_maps.out[1])) {
        return false;
    }
    AttnParams params = base_params(seq, in_layout.heads, scale);
    if (!params.status) {
        return false;
    }
    params.lse = const_cast<float *>(lse);
    params.row_dots = row_dots;
    params.out = out;
    params.dout = dout;
    params.out_ld = out_layout.ld;
    params.out_heads = out_layout.heads;
    params.dout_ld = dout_layout.ld;
    params.dout_heads = dout_layout.heads;
    if (hd == 64) {
        const size_t rows = groups * seq;
        const unsigned dots_grid =
            unsigned(std::min<size_t>((rows + 63) / 64, size_t(device_sm_count()) * 8));
        launch_chained(attention_row_dots_kernel, dots_grid, 256, 0, stream, out,
                       dout, row_dots, rows, int(seq), out_layout, dout_layout);
        ++g_kernel_launches;
    }
    AttnParams query_params = params;
    query_params.add0 = add_q ? 1 : 0;
    AttnParams key_params = params;
    key_params.add0 = add_v ? 1 : 0;
    key_params.add1 = add_k ? 1 : 0;
    if (column_partials) {
        // Rows of the partial matrix: one per CTA of either kernel's grid,
        // columns in the order of the projected gradient, [dQ | dK | dV].
        const int d_model = grad_layout.heads * hd;
        if (cudaMemsetAsync(column_partials, 0,
                            size_t(attention_tc_partial_rows()) * 3 * d_model *
                                sizeof(float),
                            stream) != cudaSuccess) {
            return false;
        }
        query_params.column_partials = key_params.column_partials = column_partials;
        query_params.partial_ld = key_params.partial_ld = 3 * d_model;
        query_params.partial_column[0] = 0;
        key_params.partial_column[0] = 2 * d_model;   // dV
        key_params.partial_column[1] = d_model;       // dK
    }
    if (hd == 32) {
        return launch<32, kGradQuery>(query_maps, query_params, groups, stream) &&
               launch<32, kGradKeyValue>(key_maps, key_params, groups, stream);
    }
    return launch<64, kGradQuery>(query_maps, query_params, groups, stream) &&
           launch<64, kGradKeyValue>(key_maps, key_params, groups, stream);
}

}  // namespace vitb200
