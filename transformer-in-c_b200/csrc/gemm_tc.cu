// Tensor-core matrix products for sm_100a: tcgen05.mma (kind::tf32, FP32
// accumulation in tensor memory) fed by TMA.
//
//   D[M,N] (+)= A[M,K] * B[K,N],  all FP32 in global memory, row-major.
//
// Either operand may be stored with the reduction index contiguous ("K-major":
// X in X*W, dY and W in dY*W^T) or with the output index contiguous
// ("MN-major": W in X*W, X and dY in X^T*dY), so the same kernel serves the
// forward product and both gradients of reference src/ops.c:107-165 without a
// transposed copy.  Nothing is converted or re-laid-out in global memory: TMA
// rounds FP32 to TF32 while it fills the shared-memory stages.
//
// Persistent CTAs (two per SM by default: with the short reductions of this
// model, K = 128..512, two shallow pipelines hide the tile-to-tile bubbles
// better than one deep one) walk work items = (128 x 128 output tile, slice
// of the reduction); three warp roles meet only through mbarriers:
//
//   warp 0      TMA producer: per 32-deep reduction block, one 128B-swizzled
//               box (K-major) or four 32x32 boxes (MN-major) per operand into
//               a shared-memory ring of 32 KB stages (2 stages by default)
//   warp 1      allocates 256 TMEM columns (two accumulators), issues four
//               K=8 tcgen05.mma per block from one lane, releases stages with
//               tcgen05.commit, and signals a finished accumulator
//   warps 2-5   epilogue, overlapped with the next item's loads and MMAs:
//               each warp tcgen05.ld's its 32 rows, adds the bias, optionally
//               derives a second output (GELU, or + residual), stages 32x32
//               blocks in its own 128B-swizzled buffers and issues its own TMA
//               stores (plain, or FP32 reduce-add for "+=" outputs and for
//               reductions split across CTAs); no block-wide barrier is used
//
// Partial tiles need no special code: TMA zero-fills out-of-range loads and
// clips out-of-range stores.  Every wait on an mbarrier is bounded in time;
// on expiry the kernel records a code in `*status` and all roles fall through
// to the common teardown, which frees the tensor memory.
#include "gemm_tc.h"
#include "kernels.h"
#include "device_util.cuh"
#include "tcgen05.cuh"

#include <cuda.h>
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <unordered_map>

namespace vitb200 {
namespace {

constexpr int kTileM = 128;
constexpr int kTileN = 128;                 // narrow tiles; the wide variant is 256
constexpr int kBlockK = 32;                 // 128 bytes of FP32 per row
constexpr int kMmaK = 8;                    // tf32 K per instruction
constexpr int kOperandBytes = kTileM * kBlockK * 4;   // 16 KiB
// Upper bound on the load ring; the launch code picks the depth that fits
// beside the epilogue staging for the chosen number of CTAs per SM.
constexpr int kMaxStages = 6;
constexpr int kSmemLimit = 227 * 1024 - 1024;   // leave room for static shared memory
constexpr int kThreads = 192;
// The tall tile has a group of four epilogue warps for each of its two
// accumulators, so that both drain at the same time.
constexpr int kThreadsTall = 320;
constexpr int kBarrierBytes = 256;   // 2 x kMaxStages + 4 mbarriers, TMEM slot

using namespace tc;

struct TcParams {
    int m, n;                 // output extents
    int k_blocks;             // ceil(reduction / 32)
    int k_blocks_per_split;
    int splits;
    int stages;               // depth of the load ring
    int staging_bytes;        // epilogue staging: 16 or 32 KiB
    int m_tiles, n_tiles;
    int a_mn_major, b_mn_major;
    int reduce_add;           // 1: TMA reduce-add into D, 0: plain store
    const float *bias;        // nullable, length n
    const float *residual;    // [m, n] with residual_pitch, for kSecondResidual
    long long residual_pitch;
    float *column_partials;   // kGeluSlope: [gridDim.x][n] column sums of D, or null
    int *status;              // device-visible word, 0 = ok
};

constexpr int kSecondGelu = 1;       // D = A*B + bias, D2 = gelu(D)
constexpr int kSecondResidual = 2;   // D = A*B + bias, D2 = D + residual
// D = (A*B) * gelu'(H): the backward pass through a GELU folded into the
// product that computes the GELU output's gradient.  H is read through
// map_d2 (one 32 x 32 block per accumulator block, by TMA into the block the
// result is then staged in); there is one output.
constexpr int kGeluSlope = 3;

// Persistent kernel: each CTA walks work items (output tile x reduction
// slice) item = blockIdx.x, blockIdx.x + gridDim.x, ...; the three roles run
// the same sequence and meet only through mbarriers, so the loads and MMAs of
// item i+1 overlap the epilogue of item i (two accumulator buffers in TMEM).
//
// TILE_N = 128: two CTAs per SM share the 512 TMEM columns (2 x 128 each).
// TILE_N = 256: one CTA per SM with all 512 columns; an MMA instruction then
// covers twice the columns for the same A bytes, which is what the
// compute-bound shapes (K >= 256) need from shared memory.  The launch code
// guarantees one CTA per SM for it through the shared-memory request, so the
// two allocations can never wait for each other.
// TILE_M = 256 (with TILE_N = 256): the tile is two 128-row halves, one
// accumulator each (all 512 columns), both multiplied by the same B tile, so
// a CTA fetches (256 + 256) x K operand values for 256 x 256 outputs: a third
// less operand traffic from L2 per multiply-add than the 128 x 256 tile, which
// is what bounds the compute-bound shapes.  The accumulators are not
// double-buffered across tiles then; instead the halves are: the epilogue
// drains half 0 while the last MMAs of half 1 run, and the next tile's MMAs
// start on half 0 while half 1 is still being drained.
// SECOND is the epilogue variant (0 or a kSecond... / kGeluSlope constant): a
// compile-time choice, so that no variant pays for another's registers.
template <int TILE_M, int TILE_N, int SECOND>
__global__ void __launch_bounds__(TILE_M == 2 * kTileM ? kThreadsTall : kThreads)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a,
               const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_d,
               const __grid_constant__ CUtensorMap map_d2, const TcParams p) {
    // All shared memory is dynamic, so that it starts at the beginning of the
    // CTA's window and the swizzled tiles get their 1024-byte alignment without
    // padding (two CTAs with three stages each fill the SM to the last KiB):
    //   [stages x 32 KiB operand tiles][epilogue staging][barriers]
    extern __shared__ __align__(1024) uint8_t smem[];
    constexpr int kHalves = TILE_M / kTileM;   // accumulators per tile
    constexpr int kABytes = TILE_M * kBlockK * 4;
    constexpr int kStageBytes = kABytes + TILE_N * kBlockK * 4;
    constexpr int kTmemColumns = 2 * TILE_N;
    static_assert(TILE_M == kTileM ||
                      (TILE_M == 2 * kTileM && (SECOND == 0 || SECOND == kSecondGelu)),
                  "the tall tile has the plain and the GELU epilogues only");
    const int kStages = p.stages;
    uint8_t *staging = smem + kStages * kStageBytes;
    uint64_t *full_bar = reinterpret_cast<uint64_t *>(staging + p.staging_bytes);
    uint64_t *empty_bar = full_bar + kMaxStages;
    uint64_t *tmem_full_bar = empty_bar + kMaxStages;
    uint64_t *tmem_empty_bar = tmem_full_bar + 2;
    uint32_t &tmem_base_slot = *reinterpret_cast<uint32_t *>(tmem_empty_bar + 2);
    uint64_t *operand_bar = tmem_empty_bar + 3;   // two per epilogue warp
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    if ((smem_address(smem) & 1023u) != 0) {
        // Never expected; without the alignment the MMA would read garbage.
        grid_dependency_wait();
        if (threadIdx.x == 0) {
            atomicExch(p.status, 6);
        }
        return;
    }

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbarrier_init(&full_bar[s], 1);
            mbarrier_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbarrier_init(&tmem_full_bar[b], 1);
            mbarrier_init(&tmem_empty_bar[b], 4);   // one arrival per epilogue warp
        }
        for (int w = 0; w < 8; ++w) {
            mbarrier_init(&operand_bar[w], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile(
            "tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::
                "r"(smem_address(&tmem_base_slot)),
            "r"(kTmemColumns)
            : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::
                         : "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    // Barriers and tensor memory are set up; from here on global memory is
    // touched, so the kernel before this one in the stream has to be complete.
    grid_dependency_wait();
    grid_dependency_release();
    const int tiles = p.m_tiles * p.n_tiles;
    const int items = tiles * p.splits;
    bool ok = true;

    if (warp == 0) {
        if (lane == 0) {
            int fill = 0;   // k-blocks loaded so far, across items
            for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
                const int tile = item % tiles;
                const int m0 = (tile / p.n_tiles) * TILE_M;
                const int n0 = (tile % p.n_tiles) * TILE_N;
                const int kb_begin = (item / tiles) * p.k_blocks_per_split;
                const int kb_end = min(p.k_blocks, kb_begin + p.k_blocks_per_split);
                for (int kb = kb_begin; kb < kb_end; ++kb, ++fill) {
                    const int s = fill % kStages;
                    const uint32_t phase = (fill / kStages) & 1;
                    ok = mbarrier_wait(&empty_bar[s], phase ^ 1);
                    if (!ok) {
                        atomicExch(p.status, 1);
                        break;
                    }
                    uint8_t *a_tile = smem + s * kStageBytes;
                    uint8_t *b_tile = a_tile + kABytes;
                    const int k0 = kb * kBlockK;
                    mbarrier_expect_tx(&full_bar[s], kStageBytes);
                    if (p.a_mn_major) {
                        for (int j = 0; j < TILE_M / 32; ++j) {
                            tma_load_2d(a_tile + j * 4096, &map_a, m0 + 32 * j, k0,
                                        &full_bar[s]);
                        }
                    } else {
                        // One box of TILE_M rows (the map's box height).
                        tma_load_2d(a_tile, &map_a, k0, m0, &full_bar[s]);
                    }
                    if (p.b_mn_major) {
                        for (int j = 0; j < TILE_N / 32; ++j) {
                            tma_load_2d(b_tile + j * 4096, &map_b, n0 + 32 * j, k0,
                                        &full_bar[s]);
                        }
                    } else {
                        tma_load_2d(b_tile, &map_b, k0, n0, &full_bar[s]);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // kind::tf32, FP32 accumulator, M = 128, N = 128.
            // (The N field is filled in per tile: a last column tile that is
            // only partly inside the matrix gets a narrower instruction.)
            const uint32_t idesc_base = (1u << 4) | (2u << 7) | (2u << 10) |
                                        (uint32_t(p.a_mn_major) << 15) |
                                        (uint32_t(p.b_mn_major) << 16) |
                                        (uint32_t(kTileM >> 4) << 24);
            // K-major: 8-row groups 1024 B apart, K steps of 32 B inside the
            // swizzled row.  MN-major: 32-wide MN atoms one box (4096 B)
            // apart, groups of four 128 B reduction rows 512 B apart, K
            // steps of eight rows.
            const uint32_t a_lead = p.a_mn_major ? 4096 : 16;
            const uint32_t b_lead = p.b_mn_major ? 4096 : 16;
            const uint32_t a_stride = p.a_mn_major ? 512 : 1024;
            const uint32_t b_stride = p.b_mn_major ? 512 : 1024;
            const uint32_t a_step = p.a_mn_major ? 1024 : kMmaK * 4;
            const uint32_t b_step = p.b_mn_major ? 1024 : kMmaK * 4;
            const uint32_t a_layout =
                p.a_mn_major ? kLayoutSwizzle128Base32 : kLayoutSwizzle128;
            const uint32_t b_layout =
                p.b_mn_major ? kLayoutSwizzle128Base32 : kLayoutSwizzle128;
            int drain = 0;   // k-blocks consumed so far, across items
            int local = 0;   // items processed by this CTA
            for (int item = blockIdx.x; item < items && ok;
                 item += gridDim.x, ++local) {
                const int tile_splits = item / tiles;
                const int n_live = min(TILE_N, p.n - ((item % tiles) % p.n_tiles) * TILE_N);
                const uint32_t idesc =
                    idesc_base | (uint32_t(((n_live + 15) & ~15) >> 3) << 17);
                const int kb_begin = tile_splits * p.k_blocks_per_split;
                const int kb_end = min(p.k_blocks, kb_begin + p.k_blocks_per_split);
                // One accumulator per tile, alternating between tiles; or, for
                // the tall tile, one per 128-row half, both used by every tile.
                const uint32_t buffer_phase =
                    kHalves == 2 ? (local & 1) : ((local >> 1) & 1);
                for (int kb = kb_begin; kb < kb_end; ++kb, ++drain) {
                    const int s = drain % kStages;
                    const uint32_t phase = (drain / kStages) & 1;
                    ok = mbarrier_wait(&full_bar[s], phase);
                    if (!ok) {
                        atomicExch(p.status, 2);
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t a_base = smem_address(smem + s * kStageBytes);
                    const uint32_t b_base = a_base + kABytes;
#pragma unroll
                    for (int h = 0; h < kHalves; ++h) {
                        const int buffer = kHalves == 2 ? h : (local & 1);
                        if (kb == kb_begin) {
                            // The epilogue must have emptied this accumulator.
                            ok = mbarrier_wait(&tmem_empty_bar[buffer],
                                               buffer_phase ^ 1);
                            if (!ok) {
                                atomicExch(p.status, 4);
                                break;
                            }
                            tcgen05_fence_after();
                        }
                        const uint32_t accumulator = tmem_base + buffer * TILE_N;
#pragma unroll
                        for (int ks = 0; ks < kBlockK / kMmaK; ++ks) {
                            const uint64_t da = operand_descriptor(
                                a_base + h * kOperandBytes + ks * a_step, a_lead,
                                a_stride, a_layout);
                            const uint64_t db = operand_descriptor(
                                b_base + ks * b_step, b_lead, b_stride, b_layout);
                            tcgen05_mma_tf32(accumulator, da, db, idesc,
                                             (kb > kb_begin || ks > 0) ? 1u : 0u);
                        }
                        if (kb == kb_end - 1) {
                            // This half is complete: its rows can leave while
                            // the other half's last products still run.
                            tcgen05_commit(&tmem_full_bar[buffer]);
                        }
                    }
                    if (!ok) {
                        break;
                    }
                    tcgen05_commit(&empty_bar[s]);
                }
            }
        }
    } else if constexpr (SECOND == kGeluSlope) {
        // Epilogue of D = (A*B) * gelu'(H).  Each warp walks its 32 x 32
        // blocks in order (tile after tile, four column chunks per tile) as a
        // two-deep pipeline over its two staging blocks: while block j is
        // multiplied and stored, the copy engine already fetches the H values
        // of block j+1 into the other staging block, so the latency of that
        // read stays off the critical path.
        const int quarter = warp & 3;
        uint8_t *my_staging = staging + quarter * (p.staging_bytes / 4);
        uint64_t *my_bar = operand_bar + 2 * quarter;
        uint32_t phases = 0;   // bit b: parity of the next completion of my_bar[b]
        int issued = 0;        // H blocks requested so far
        int consumed = 0;      // H blocks used so far
        // Requests the H block of (item, chunk) when that block exists.
        auto request = [&](int item, int chunk) {
            const int tile = item % tiles;
            const int m0 = (tile / p.n_tiles) * kTileM + quarter * 32;
            const int col0 = (tile % p.n_tiles) * TILE_N + chunk * 32;
            if (col0 >= p.n || m0 >= p.m) {
                return;
            }
            if (lane == 0) {
                // The block was last read by the store issued for the block
                // before the current one.
                asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                const int b = issued & 1;
                mbarrier_expect_tx(&my_bar[b], 4096);
                tma_load_2d(my_staging + b * 4096, &map_d2, col0, m0, &my_bar[b]);
            }
            ++issued;
        };
        if (int(blockIdx.x) < items) {
            request(blockIdx.x, 0);
        }
        int local = 0;
        for (int item = blockIdx.x; item < items && ok; item += gridDim.x, ++local) {
            const int tile = item % tiles;
            const int m0 = (tile / p.n_tiles) * kTileM + quarter * 32;
            const int n0 = (tile % p.n_tiles) * TILE_N;
            const int buffer = local & 1;
            const uint32_t buffer_phase = (local >> 1) & 1;
            ok = mbarrier_wait(&tmem_full_bar[buffer], buffer_phase);
            ok = __all_sync(0xffffffffu, ok);   // keep the warp in step
            if (!ok) {
                atomicExch(p.status, 3);
                break;
            }
            tcgen05_fence_after();
#pragma unroll 1
            for (int chunk = 0; chunk < TILE_N / 32; ++chunk) {
                const int col0 = n0 + chunk * 32;
                const bool chunk_live = col0 < p.n && m0 < p.m;
                uint32_t r[32];
                if (chunk_live) {
                    tcgen05_load_32(tmem_base + (uint32_t(quarter * 32) << 16) +
                                        buffer * TILE_N + chunk * 32,
                                    r);
                }
                if (chunk == TILE_N / 32 - 1) {
                    tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        mbarrier_arrive(&tmem_empty_bar[buffer]);
                    }
                }
                // The block after this one, possibly the next tile's first.
                if (chunk + 1 < TILE_N / 32) {
                    request(item, chunk + 1);
                } else if (item + int(gridDim.x) < items) {
                    request(item + gridDim.x, 0);
                }
                if (!chunk_live) {
                    continue;   // uniform across the warp
                }
                const int b = consumed & 1;
                ++consumed;
                ok = mbarrier_wait(&my_bar[b], (phases >> b) & 1u);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) {
                    atomicExch(p.status, 7);
                    break;
                }
                phases ^= 1u << b;
                float *block = reinterpret_cast<float *>(my_staging + b * 4096);
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    // 128-byte swizzle: 16-byte chunk c of row r lives at
                    // chunk position c ^ (r % 8).
                    const int offset = lane * 32 + 4 * (c ^ (lane & 7));
                    float4 h = *reinterpret_cast<const float4 *>(block + offset);
                    h.x = __uint_as_float(r[4 * c + 0]) * gelu_slope_fast(h.x);
                    h.y = __uint_as_float(r[4 * c + 1]) * gelu_slope_fast(h.y);
                    h.z = __uint_as_float(r[4 * c + 2]) * gelu_slope_fast(h.z);
                    h.w = __uint_as_float(r[4 * c + 3]) * gelu_slope_fast(h.w);
                    *reinterpret_cast<float4 *>(block + offset) = h;
                }
                if (p.column_partials) {
                    // Column sums of the block (rows past the matrix are
                    // zero: their accumulators are), lane = column.
                    __syncwarp();
                    float sum = 0.0f;
#pragma unroll
                    for (int row = 0; row < 32; ++row) {
                        sum += block[row * 32 + 4 * ((lane >> 2) ^ (row & 7)) +
                                     (lane & 3)];
                    }
                    if (col0 + lane < p.n) {
                        atomicAdd(p.column_partials + size_t(blockIdx.x) * p.n +
                                      col0 + lane,
                                  sum);
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) {
                    tma_store_2d(block, &map_d, col0, m0);
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
            }
        }
        if (lane == 0) {
            asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        }
    } else {
        // Epilogue warps 2..5 own TMEM lane quarters 2, 3, 0, 1, i.e. 32 rows
        // of the tile each.  A warp stages its own 32 x 32 blocks (4 KiB, two
        // buffers per output) and issues its own TMA stores, so the epilogue
        // needs no block-wide barrier at all.
        const int quarter = warp & 3;
        const int outputs = SECOND ? 2 : 1;
        // Per warp: two 4 KiB blocks (one output double-buffered, or one buffer
        // for each of two outputs), or a single block when the load ring was
        // given the space instead.
        // The tall tile: warps 2-5 drain the upper half's accumulator, warps
        // 6-9 the lower half's, each warp through one 4 KiB block.
        const int half = kHalves == 2 ? (warp - 2) >> 2 : 0;
        const int buffers =
            kHalves == 2 ? 1 : (outputs == 2 ? 1 : p.staging_bytes / (4 * 4096));
        uint8_t *my_staging = kHalves == 2
            ? staging + (warp - 2) * 4096
            : staging + quarter * (p.staging_bytes / 4);
        int local = 0;
        int stored = 0;   // blocks handed to TMA so far (selects the buffer)
        for (int item = blockIdx.x; item < items; item += gridDim.x, ++local) {
            const int tile = item % tiles;
            const int m0 = (tile / p.n_tiles) * TILE_M + half * kTileM + quarter * 32;
            const int n0 = (tile % p.n_tiles) * TILE_N;
            const int buffer = kHalves == 2 ? half : (local & 1);
            const uint32_t buffer_phase =
                kHalves == 2 ? (local & 1) : ((local >> 1) & 1);
            ok = mbarrier_wait(&tmem_full_bar[buffer], buffer_phase);
            ok = __all_sync(0xffffffffu, ok);   // keep the warp in step
            if (!ok) {
                atomicExch(p.status, 3);
                break;
            }
            tcgen05_fence_after();
#pragma unroll 1
            for (int chunk = 0; chunk < TILE_N / 32; ++chunk) {
                const int col0 = n0 + chunk * 32;
                const bool chunk_live = col0 < p.n && m0 < p.m;
                // Bias for these 32 columns, requested before the accumulator
                // so the two latencies overlap.
                float4 bias[8];
                if (p.bias && chunk_live) {
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        const int col = col0 + 4 * c;
                        if (col + 3 < p.n) {
                            bias[c] = __ldg(
                                reinterpret_cast<const float4 *>(p.bias + col));
                        } else {
                            bias[c].x = col + 0 < p.n ? __ldg(p.bias + col + 0) : 0.f;
                            bias[c].y = col + 1 < p.n ? __ldg(p.bias + col + 1) : 0.f;
                            bias[c].z = col + 2 < p.n ? __ldg(p.bias + col + 2) : 0.f;
                            bias[c].w = 0.f;
                        }
                    }
                }
                uint32_t r[32];
                if (chunk_live) {
                    tcgen05_load_32(tmem_base + (uint32_t(quarter * 32) << 16) +
                                        buffer * TILE_N + chunk * 32,
                                    r);
                }
                if (chunk == TILE_N / 32 - 1) {
                    // Everything this warp needs is in registers: hand the
                    // accumulator buffer back to the MMA warp.
                    tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        mbarrier_arrive(&tmem_empty_bar[buffer]);
                    }
                }
                if (!chunk_live) {
                    continue;   // uniform across the warp
                }
                if (p.bias) {
                    // Folded into the accumulator registers once, so the bias
                    // registers are free again before the stores.
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        r[4 * c + 0] = __float_as_uint(__uint_as_float(r[4 * c + 0]) + bias[c].x);
                        r[4 * c + 1] = __float_as_uint(__uint_as_float(r[4 * c + 1]) + bias[c].y);
                        r[4 * c + 2] = __float_as_uint(__uint_as_float(r[4 * c + 2]) + bias[c].z);
                        r[4 * c + 3] = __float_as_uint(__uint_as_float(r[4 * c + 3]) + bias[c].w);
                    }
                }
                // The buffer about to be rewritten was last read by the store
                // this warp issued two blocks ago.
                if (lane == 0) {
                    if (buffers == 2) {
                        asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                    } else {
                        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                    }
                }
                __syncwarp();
                const int slot = buffers == 2 ? (stored & 1) : 0;
                ++stored;
                float *first = reinterpret_cast<float *>(my_staging + slot * 4096);
                // With 16 KiB of staging both outputs of a warp go through the
                // same 4 KiB block, one after the other.
                const bool shared_block =
                    outputs == 2 && (kHalves == 2 || p.staging_bytes == kOperandBytes);
                float *second = shared_block
                    ? first : reinterpret_cast<float *>(my_staging + 4096);
                {
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    float4 v;
                    v.x = __uint_as_float(r[4 * c + 0]);
                    v.y = __uint_as_float(r[4 * c + 1]);
                    v.z = __uint_as_float(r[4 * c + 2]);
                    v.w = __uint_as_float(r[4 * c + 3]);
                    // 128-byte swizzle: 16-byte chunk c of row r lives at
                    // chunk position c ^ (r % 8).
                    const int offset = lane * 32 + 4 * (c ^ (lane & 7));
                    *reinterpret_cast<float4 *>(first + offset) = v;
                    if (SECOND == kSecondGelu && !shared_block) {
                        v.x = gelu_value_fast(v.x);
                        v.y = gelu_value_fast(v.y);
                        v.z = gelu_value_fast(v.z);
                        v.w = gelu_value_fast(v.w);
                        *reinterpret_cast<float4 *>(second + offset) = v;
                    }
                }
                }
                if (SECOND == kSecondResidual) {
                    // D2 = D + residual.  In the accumulator layout a lane
                    // owns a row, which would read the residual one row per
                    // lane; instead the staged block is walked with eight
                    // lanes per row, so every load covers four full 128-byte
                    // row segments.
                    __syncwarp();
                    const int c = lane & 7;
                    const int col = col0 + 4 * c;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int row = (lane >> 3) + 4 * i;
                        const int offset = row * 32 + 4 * (c ^ (row & 7));
                        float4 v = *reinterpret_cast<const float4 *>(first + offset);
                        if (m0 + row < p.m) {
                            const float *res = p.residual +
                                size_t(m0 + row) * p.residual_pitch + col;
                            if (col + 3 < p.n) {
                                const float4 x =
                                    __ldcs(reinterpret_cast<const float4 *>(res));
                                v.x += x.x; v.y += x.y; v.z += x.z; v.w += x.w;
                            } else {
                                if (col + 0 < p.n) v.x += res[0];
                                if (col + 1 < p.n) v.y += res[1];
                                if (col + 2 < p.n) v.z += res[2];
                            }
                        }
                        *reinterpret_cast<float4 *>(second + offset) = v;
                    }
                }
                // Make the generic-proxy writes visible to the TMA engine.
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (shared_block && SECOND == kSecondGelu) {
                    // First output out; the second output's values are
                    // computed while the copy engine reads the block, and go
                    // through the same block once it has.
                    if (lane == 0) {
                        tma_store_2d(first, &map_d, col0, m0);
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
#pragma unroll
                    for (int e = 0; e < 32; ++e) {
                        r[e] = __float_as_uint(gelu_value_fast(__uint_as_float(r[e])));
                    }
                    if (lane == 0) {
                        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                    }
                    __syncwarp();
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        float4 v;
                        v.x = __uint_as_float(r[4 * c + 0]);
                        v.y = __uint_as_float(r[4 * c + 1]);
                        v.z = __uint_as_float(r[4 * c + 2]);
                        v.w = __uint_as_float(r[4 * c + 3]);
                        const int offset = lane * 32 + 4 * (c ^ (lane & 7));
                        *reinterpret_cast<float4 *>(second + offset) = v;
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(second, &map_d2, col0, m0);
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                } else if (lane == 0) {
                    if (p.reduce_add) {
                        tma_reduce_add_2d(first, &map_d, col0, m0);
                    } else {
                        tma_store_2d(first, &map_d, col0, m0);
                    }
                    if (outputs == 2) {
                        tma_store_2d(second, &map_d2, col0, m0);
                    }
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(
                         tmem_base),
                     "r"(kTmemColumns)
                     : "memory");
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
    unsigned long long inner, outer, pitch;
    unsigned box_inner, box_outer;
    int swizzle;
    bool operator==(const MapKey &o) const {
        return base == o.base && inner == o.inner && outer == o.outer &&
               pitch == o.pitch && box_inner == o.box_inner &&
               box_outer == o.box_outer && swizzle == o.swizzle;
    }
};

struct MapKeyHash {
    size_t operator()(const MapKey &k) const {
        size_t h = reinterpret_cast<size_t>(k.base);
        h = h * 1000003u ^ k.inner;
        h = h * 1000003u ^ k.outer;
        h = h * 1000003u ^ k.pitch;
        h = h * 1000003u ^ (size_t(k.box_inner) << 16 | k.box_outer);
        h = h * 1000003u ^ size_t(k.swizzle);
        return h;
    }
};

// 2-D FP32 tensor map over a row-major matrix: `inner` contiguous elements per
// row, `outer` rows `pitch` elements apart, with the given 128-byte swizzle
// flavour.  Operand maps use the TFLOAT32 element type, which makes the copy
// engine round the FP32 words to TF32 (nearest) on their way into shared
// memory instead of leaving the truncation to the MMA; the output map is plain
// FP32.  Encoded maps are cached: the training step presents the same buffers
// every iteration.
bool tensor_map(const float *base, unsigned long long inner,
                unsigned long long outer, unsigned long long pitch,
                unsigned box_inner, unsigned box_outer,
                CUtensorMapSwizzle swizzle, bool as_tf32, CUtensorMap *out) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    const MapKey key{base, inner, outer, pitch, box_inner, box_outer,
                     int(swizzle) * 2 + int(as_tf32)};
    auto found = cache.find(key);
    if (found != cache.end()) {
        *out = found->second;
        return true;
    }
    EncodeTiled encode = encode_tiled();
    if (!encode) {
        return false;
    }
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {pitch * sizeof(float)};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t element_strides[2] = {1, 1};
    const CUresult status = encode(
        out, as_tf32 ? CU_TENSOR_MAP_DATA_TYPE_TFLOAT32
                     : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(base), dims,
        strides, box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
        swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (status != CUDA_SUCCESS) {
        return false;
    }
    if (cache.size() > 4096) {
        cache.clear();
    }
    cache.emplace(key, *out);
    return true;
}

int *status_word() {
    static int *word = []() -> int * {
        int *memory = nullptr;
        if (cudaHostAlloc(reinterpret_cast<void **>(&memory), sizeof(int),
                          cudaHostAllocMapped) != cudaSuccess) {
            return nullptr;
        }
        *memory = 0;
        return memory;
    }();
    return word;
}

}  // namespace

bool gemm_tc_supported(const TcGemm &g) {
    // TMA needs 16-byte aligned bases and row pitches.  An extent may be
    // smaller than the 32-wide box (the 16-pixel patches of the 28 x 28
    // models): out-of-range elements load as zero and stores are clipped.
    // Tiny extents are left to the FP32 kernel.
    auto aligned = [](const void *p) {
        return (reinterpret_cast<uintptr_t>(p) & 15) == 0;
    };
    return g.m >= 16 && g.n >= 16 && g.k >= 16 && g.lda % 4 == 0 &&
           g.ldb % 4 == 0 && g.ldd % 4 == 0 && aligned(g.a) && aligned(g.b) &&
           aligned(g.d) && (!g.bias || aligned(g.bias)) &&
           (!g.d2 || (aligned(g.d2) && g.ldd2 % 4 == 0 && !g.accumulate)) &&
           (!g.residual || (aligned(g.residual) && g.ld_residual % 4 == 0)) &&
           (!g.gelu_input ||
            (aligned(g.gelu_input) && g.ld_gelu_input % 4 == 0 && !g.accumulate &&
             !g.bias && !g.d2)) &&
           (!g.column_partials || g.gelu_input) &&
           status_word() &&
           encode_tiled();
}

int launch_gemm_tc(const TcGemm &g, cudaStream_t stream) {
    if (!gemm_tc_supported(g)) {
        return -1;
    }
    static bool configured = false;
    if (!configured) {
        const void *kernels[] = {
            reinterpret_cast<const void *>(gemm_tc_kernel<128, 128, 0>),
            reinterpret_cast<const void *>(gemm_tc_kernel<128, 128, kSecondGelu>),
            reinterpret_cast<const void *>(gemm_tc_kernel<128, 128, kSecondResidual>),
            reinterpret_cast<const void *>(gemm_tc_kernel<128, 128, kGeluSlope>),
            reinterpret_cast<const void *>(gemm_tc_kernel<128, 256, 0>),
            reinterpret_cast<const void *>(gemm_tc_kernel<128, 256, kSecondGelu>),
            reinterpret_cast<const void *>(gemm_tc_kernel<256, 256, 0>),
            reinterpret_cast<const void *>(gemm_tc_kernel<256, 256, kSecondGelu>)};
        for (const void *kernel : kernels) {
            if (cudaFuncSetAttribute(kernel,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     kSmemLimit) != cudaSuccess) {
                return -1;
            }
        }
        configured = true;
    }
    // Wide tiles where the product is compute-bound: deep reductions, one
    // output (or the GELU pair), a multiple of 128 columns.
    static const int forced_tile =
        getenv("VITB200_TC_TILE_N") ? atoi(getenv("VITB200_TC_TILE_N")) : 0;
    const bool gelu_pair = g.d2 && !g.residual;
    // (A last tile that is half outside the matrix costs half: its products
    // are issued 128 columns wide.)
    // That pays from 4.5 tiles on, or with a deep reduction (measured at
    // [65600,384]x[384,1152]: +14 %, [65600,1536]x[1536,384]: +6 %,
    // [65600,384]x[384,384]: -3 to -9 %).
    const bool divides = g.n % 256 == 0 ||
                         (g.n % 128 == 0 && g.n >= 256 &&
                          (g.n >= 1024 || (!g.accumulate && g.k >= 1024)));
    bool wide = (!g.d2 || gelu_pair) && !g.gelu_input && g.k >= 256 && divides;
    if (forced_tile == 128 || (g.d2 && !gelu_pair) || g.gelu_input) {
        wide = false;
    } else if (forced_tile == 256 && !g.d2) {
        wide = g.n >= 256;
    }
    // Tall tiles (256 x 256, two accumulator halves) on top of that when there
    // are at least two full row tiles: a third less operand traffic from L2.
    static const int forced_tile_m =
        getenv("VITB200_TC_TILE_M") ? atoi(getenv("VITB200_TC_TILE_M")) : 0;
    // (Not for the shortest reductions, where the double-buffered 128 x 256
    // tile hides its epilogue completely and measured a few percent better.)
    const bool long_enough = g.accumulate || g.k >= 384;
    // A last row tile that is half empty costs a full one: only where that
    // is a small share of the rows.
    const bool fits = g.m % (2 * kTileM) == 0 || g.m % (2 * kTileM) > kTileM ||
                      g.m >= 16 * kTileM;
    bool tall = wide && g.m >= 2 * kTileM && forced_tile_m != 128 &&
                ((long_enough && fits) || forced_tile_m == 256);
    // The GELU pair's epilogue (two stores and a GELU per element) takes
    // longer than the tile's products: the tall tile, whose accumulators are
    // not double-buffered across tiles, leaves it exposed; the 128 x 256 tile
    // hides the next tile's products behind it (measured 3 to 10 % faster at
    // [100864,512]x[512,2048] and [65600,384]x[384,1536]).
    static const bool gelu_pair_tall = getenv("VITB200_TC_GELU_TALL") != nullptr;
    if (gelu_pair && tall && !gelu_pair_tall) {
        tall = false;
    }
    if (gelu_pair && !long_enough) {
        // Short reductions: two CTAs per SM on 128 x 128 tiles measured
        // better (0.192 against 0.204 ms at [100864,256]x[256,1024]).
        wide = false;
    }
    const int tile_n = wide ? 256 : kTileN;
    const int tile_m = tall ? 2 * kTileM : kTileM;
    CUtensorMap map_a, map_b, map_d;
    // K-major operand: rows = output index, inner = reduction index.
    // MN-major operand: rows = reduction index, inner = output index.
    const CUtensorMapSwizzle chunks16 = CU_TENSOR_MAP_SWIZZLE_128B;
    const CUtensorMapSwizzle chunks32 = CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B;
    const bool ok_a = g.a_mn_major
        ? tensor_map(g.a, g.m, g.k, g.lda, 32, 32, chunks32, true, &map_a)
        : tensor_map(g.a, g.k, g.m, g.lda, 32, tile_m, chunks16, true, &map_a);
    const bool ok_b = g.b_mn_major
        ? tensor_map(g.b, g.n, g.k, g.ldb, 32, 32, chunks32, true, &map_b)
        : tensor_map(g.b, g.k, g.n, g.ldb, 32, tile_n, chunks16, true, &map_b);
    const bool ok_d =
        tensor_map(g.d, g.n, g.m, g.ldd, 32, 32, chunks16, false, &map_d);
    CUtensorMap map_d2 = map_d;
    const bool ok_d2 = !g.d2 ||
        tensor_map(g.d2, g.n, g.m, g.ldd2, 32, 32, chunks16, false, &map_d2);
    if (!ok_a || !ok_b || !ok_d || !ok_d2) {
        return -1;
    }
    if (g.gelu_input &&
        !tensor_map(g.gelu_input, g.n, g.m, g.ld_gelu_input, 32, 32, chunks16,
                    false, &map_d2)) {
        return -1;
    }
    TcParams p;
    p.m = g.m;
    p.n = g.n;
    p.k_blocks = (g.k + kBlockK - 1) / kBlockK;
    p.n_tiles = (g.n + tile_n - 1) / tile_n;
    const int m_tiles = (g.m + tile_m - 1) / tile_m;
    p.m_tiles = m_tiles;
    const int tiles = m_tiles * p.n_tiles;
    // Two persistent CTAs per SM, each with a 2-stage load ring and 32 KiB of
    // epilogue staging (97 KiB): they interleave their MMA issue and their
    // epilogues, and measured faster than one CTA with a 4- to 6-stage ring
    // at every size tried (449 against 346 TFLOP/s at [100864,512]x[512,2048]).
    // A single output can give up the second staging buffer of each epilogue
    // warp for a third load stage: more bytes in flight, which is what the
    // short-K, bandwidth-bound products of this model lack.
    int staging_bytes = 2 * kOperandBytes;
    int ctas_per_sm = 2;
    p.stages = 2;
    if ((!g.d2 || !g.residual) && !g.gelu_input) {
        // (Also the GELU pair: its two outputs share each warp's block.)
        p.stages = 3;
        staging_bytes = kOperandBytes;
    }
    static const int forced_staging =
        getenv("VITB200_TC_STAGING") ? atoi(getenv("VITB200_TC_STAGING")) : 0;
    static const int forced_stages =
        getenv("VITB200_TC_STAGES") ? atoi(getenv("VITB200_TC_STAGES")) : 0;
    static const int forced_ctas =
        getenv("VITB200_TC_CTAS") ? atoi(getenv("VITB200_TC_CTAS")) : 0;
    if (forced_stages > 0 && forced_stages <= kMaxStages) {
        p.stages = forced_stages;
    }
    if (forced_ctas > 0) {
        ctas_per_sm = forced_ctas;
    }
    if (wide) {
        // One CTA per SM (it owns all of tensor memory): four 48 KiB stages
        // and double-buffered staging, 224 KiB.
        ctas_per_sm = 1;
        p.stages = tall ? 3 : 4;   // 64 KiB stages when the tile is tall
        staging_bytes = 2 * kOperandBytes;
    }
    if (forced_staging == 1 && !(g.d2 && g.residual)) {
        staging_bytes = kOperandBytes;
    } else if (forced_staging == 2 || (forced_stages > 0 && forced_staging == 0)) {
        staging_bytes = 2 * kOperandBytes;
    }
    if (g.gelu_input) {
        staging_bytes = 2 * kOperandBytes;   // its epilogue pipeline needs both blocks
        if (p.stages > 2 && ctas_per_sm > 1) {
            p.stages = 2;
        }
    }
    p.staging_bytes = staging_bytes;
    // One or two persistent CTAs on every multiprocessor (never more than
    // the per-CTA partial rows provide for).
    const long long slots =
        std::min<long long>((long long)device_sm_count() * ctas_per_sm, kGemmPartialRows);
    int splits = 1;
    if (g.accumulate) {
        // Long reductions onto few output tiles (weight gradients) are cut
        // into slices.  With a persistent grid the slices should fill the CTA
        // slots evenly: pick the slice count that minimises the k-blocks the
        // busiest CTA walks, charging each item about eight k-blocks for its
        // epilogue and reduce-add.
        long long best_cost = -1;
        for (int candidate = 1; candidate <= 512; ++candidate) {
            const int per_slice = (p.k_blocks + candidate - 1) / candidate;
            if (candidate > 1 && per_slice < 4) {
                break;
            }
            const long long rounds =
                ((long long)tiles * candidate + slots - 1) / slots;
            const long long cost = rounds * (per_slice + 8);
            if (best_cost < 0 || cost < best_cost) {
                best_cost = cost;
                splits = candidate;
            }
        }
    }
    p.k_blocks_per_split = (p.k_blocks + splits - 1) / splits;
    splits = (p.k_blocks + p.k_blocks_per_split - 1) / p.k_blocks_per_split;
    p.a_mn_major = g.a_mn_major ? 1 : 0;
    p.b_mn_major = g.b_mn_major ? 1 : 0;
    p.reduce_add = g.accumulate ? 1 : 0;
    p.bias = g.bias;
    const int second = g.d2 ? (g.residual ? kSecondResidual : kSecondGelu)
                            : (g.gelu_input ? kGeluSlope : 0);
    p.column_partials = g.column_partials;
    p.residual = g.residual;
    p.residual_pitch = g.ld_residual;
    int *device_status = nullptr;
    cudaHostGetDevicePointer(reinterpret_cast<void **>(&device_status),
                             status_word(), 0);
    p.status = device_status;
    p.splits = splits;
    // One persistent CTA per SM (the shared-memory ring fills an SM), fewer
    // when there is less work than SMs.
    const long long items = (long long)tiles * splits;
    const int stage_bytes = (tile_m + tile_n) * kBlockK * 4;
    const int smem_bytes = p.stages * stage_bytes + staging_bytes + kBarrierBytes;
    const unsigned grid = unsigned(items < slots ? items : slots);
    if (g.column_partials && grid > unsigned(kGemmPartialRows)) {
        return -1;
    }
    if (g.column_partials) {
        if (cudaMemsetAsync(g.column_partials, 0,
                            size_t(kGemmPartialRows) * g.n * sizeof(float),
                            stream) != cudaSuccess) {
            return -1;
        }
    }
    if (tall && second == kSecondGelu) {
        launch_chained(gemm_tc_kernel<256, 256, kSecondGelu>, grid,
                       kThreadsTall, smem_bytes, stream, map_a, map_b, map_d,
                       map_d2, p);
    } else if (tall) {
        launch_chained(gemm_tc_kernel<256, 256, 0>, grid, kThreadsTall,
                       smem_bytes, stream, map_a, map_b, map_d, map_d2, p);
    } else if (wide && second == kSecondGelu) {
        launch_chained(gemm_tc_kernel<128, 256, kSecondGelu>, grid, kThreads,
                       smem_bytes, stream, map_a, map_b, map_d, map_d2, p);
    } else if (wide) {
        launch_chained(gemm_tc_kernel<128, 256, 0>, grid, kThreads, smem_bytes,
                       stream, map_a, map_b, map_d, map_d2, p);
    } else if (second == kSecondGelu) {
        launch_chained(gemm_tc_kernel<128, 128, kSecondGelu>, grid, kThreads,
                       smem_bytes, stream, map_a, map_b, map_d, map_d2, p);
    } else if (second == kSecondResidual) {
        launch_chained(gemm_tc_kernel<128, 128, kSecondResidual>, grid,
                       kThreads, smem_bytes, stream, map_a, map_b, map_d,
                       map_d2, p);
    } else if (second == kGeluSlope) {
        launch_chained(gemm_tc_kernel<128, 128, kGeluSlope>, grid, kThreads,
                       smem_bytes, stream, map_a, map_b, map_d, map_d2, p);
    } else {
        launch_chained(gemm_tc_kernel<128, 128, 0>, grid, kThreads, smem_bytes,
                       stream, map_a, map_b, map_d, map_d2, p);
    }
    ++g_kernel_launches;
    ++g_tc_products;
    if (wide) {
        ++g_tc_wide_products;
    }
    return 0;
}

unsigned long long g_tc_products = 0, g_tc_wide_products = 0;

int gemm_tc_status() {
    int *word = status_word();
    return word ? *word : 0;
}

int *tc_status_device_pointer() {
    int *word = status_word();
    int *device = nullptr;
    if (!word || cudaHostGetDevicePointer(reinterpret_cast<void **>(&device),
                                          word, 0) != cudaSuccess) {
        return nullptr;
    }
    return device;
}

}  // namespace vitb200
