// Tensor-core attention for sequences of at most 64 tokens: the whole
// (sample, head) group is one 64 x 64 score tile, and everything between the
// operand tiles and the results stays in registers.
//
// Same mathematics as the FP32 kernels (reference src/ops.c:1297-1355 forward,
// :1381-1441 backward) on warp-level mma.sync m16n8k8 with TF32 operands
// rounded to nearest and FP32 accumulation.  A block of two warps serves one
// group; a warp owns 16-row tiles of the result.  The operand matrices
// (K, V for the forward pass; Q, K, V, dO for the backward pass) are staged in
// shared memory once, already rounded; no score, probability or gradient tile
// ever goes to shared memory:
//
//  * The accumulator layout of one product is turned into the A operand of
//    the next (P -> P V, dS -> dS K, P^T -> P^T dO, dS^T -> dS^T Q) without
//    moving data between lanes.  A lane holds columns 2t and 2t+1 of every
//    8-column accumulator tile; an A fragment wants columns t and t+4.  The
//    sum over the contraction index does not care about its order, so the
//    lane's two columns are declared to be "t" and "t+4" and the B operand's
//    rows are fetched in the matching order (rows 8s+2t and 8s+2t+1).
//  * The same freedom on the head dimension lets every fragment be fetched
//    with 64- or 128-bit shared-memory loads: lane t owns HD/4 consecutive
//    floats of a row and feeds them to the k-steps two at a time.
//  * The backward pass needs P and dS transposed for dV and dK.  Instead of
//    transposing through shared memory it recomputes the transposed tiles
//    from swapped operands (S^T = K Q^T, dP^T = V dO^T) and normalises them
//    with the per-row log-sum-exp and D = dO.O values of the first pass, the
//    only data exchanged between the two warps (128 floats).
//
// Operands and results are addressed through HeadLayout, so the kernels read
// Q, K, V straight out of the projected matrix and write into the merged /
// projected-gradient matrices when the caller fuses the head regrouping.
#include "kernels.h"
#include "device_util.cuh"

#include <cfloat>
#include <cstdint>

namespace vitb200 {
namespace {

constexpr int kTile = 64;       // rows of every staged operand tile
constexpr int kWarps = 2;
constexpr int kThreads = kWarps * 32;
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float to_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}

__device__ __forceinline__ float exp2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void mma_tf32(float (&c)[4], float a0, float a1,
                                         float a2, float a3, float b0,
                                         float b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 "
        "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(__float_as_uint(a0)), "r"(__float_as_uint(a1)),
          "r"(__float_as_uint(a2)), "r"(__float_as_uint(a3)),
          "r"(__float_as_uint(b0)), "r"(__float_as_uint(b1)));
}

__device__ __forceinline__ float quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(kFullMask, v, 1));
    return fmaxf(v, __shfl_xor_sync(kFullMask, v, 2));
}

__device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(kFullMask, v, 1);
    return v + __shfl_xor_sync(kFullMask, v, 2);
}

template <int HD>
struct Shape {
    // Floats a staged tile row takes: four floats of padding keep the fragment
    // loads of head dimension 32 apart; 16 and 64 use a swizzle instead
    // (tile_index).
    static constexpr int kPitch = HD == 16 ? 16 : (HD == 64 ? 64 : HD + 4);
    static constexpr int kRange = HD / 4;     // floats of a row one lane owns
    static constexpr int kSteps = HD / 8;     // k-steps over the head dimension
    static constexpr int kOut = HD / 8;       // 8-column tiles of an HD-wide result
};

// Where element (row, col) of a staged tile lives.  Head dimension 16: rows of
// 64 bytes, no padding; each pair of rows fills the 32 banks once, the second
// pair of every four rows is stored in swapped order and rows 4..7 of every
// eight swap their 32-byte halves.  With that both access patterns of the
// products are free of bank conflicts: the 128-bit loads of product_rows
// (eight lanes = two consecutive rows) and the 64-bit loads of
// product_columns (sixteen lanes = four rows two apart, a 32-byte quarter of
// each), which padding alone cannot give at this width.
template <int HD>
__host__ __device__ __forceinline__ int tile_index(int row, int col) {
    if (HD == 16) {
        const int slot = (row & ~1) | ((row ^ (row >> 1)) & 1);
        const int chunk = (col >> 2) ^ ((row >> 1) & 2);
        return slot * 16 + (chunk << 2) + (col & 3);
    }
    if (HD == 64) {
        // Rows of 256 bytes (sixteen 16-byte chunks, two passes over the
        // banks), the chunk index XORed with a row-dependent value out of
        // {0, 1, 4, 5}: bit 2 separates the two consecutive rows that one
        // 128-bit load of product_rows touches (its lanes read four adjacent
        // chunks each, see lane_column), bits 0 and 2 spread the four rows two
        // apart of one load of product_columns (two chunks each) over the
        // eight bank groups.  With a padded pitch either pattern is left with
        // a two-way conflict.
        const int twist = ((row >> 1) & 1) | ((((row >> 2) ^ row) & 1) << 2);
        return row * 64 + ((((col >> 2) ^ twist)) << 2) + (col & 3);
    }
    return row * Shape<HD>::kPitch + col;
}

// Column of element e of the head-dimension slice lane t contracts over (the
// A rows and B rows of product_rows).  Any split of the columns over the four
// lanes works as long as both operands use the same one: consecutive quarters
// in general; at head dimension 64 the lane takes every fourth 16-byte chunk,
// so that the four lanes of a row read adjacent chunks of shared memory.
template <int HD>
__host__ __device__ __forceinline__ int lane_column(int t, int e) {
    if (HD == 64) {
        return (e >> 2) * 16 + t * 4 + (e & 3);
    }
    return t * Shape<HD>::kRange + e;
}

// The lane's slice of a row in global memory (row points at column 0).
template <int HD>
__device__ __forceinline__ void load_lane_global(float (&x)[HD / 4],
                                                 const float *row, int t,
                                                 bool rounded) {
#pragma unroll
    for (int i = 0; i < HD / 4; i += 4) {
        const float4 v = __ldcs(
            reinterpret_cast<const float4 *>(row + lane_column<HD>(t, i)));
        x[i] = rounded ? to_tf32(v.x) : v.x;
        x[i + 1] = rounded ? to_tf32(v.y) : v.y;
        x[i + 2] = rounded ? to_tf32(v.z) : v.z;
        x[i + 3] = rounded ? to_tf32(v.w) : v.w;
    }
}

// The lane's kRange consecutive floats of a row (16-byte aligned).
template <int N>
__device__ __forceinline__ void load_range(float (&x)[N], const float *source) {
#pragma unroll
    for (int i = 0; i < N; i += 4) {
        const float4 v = *reinterpret_cast<const float4 *>(source + i);
        x[i] = v.x; x[i + 1] = v.y; x[i + 2] = v.z; x[i + 3] = v.w;
    }
}

template <int N>
__device__ __forceinline__ void load_range_global(float (&x)[N],
                                                  const float *source,
                                                  bool rounded) {
#pragma unroll
    for (int i = 0; i < N; i += 4) {
        const float4 v = __ldcs(reinterpret_cast<const float4 *>(source + i));
        x[i] = rounded ? to_tf32(v.x) : v.x;
        x[i + 1] = rounded ? to_tf32(v.y) : v.y;
        x[i + 2] = rounded ? to_tf32(v.z) : v.z;
        x[i + 3] = rounded ? to_tf32(v.w) : v.w;
    }
}

// Staging of rows [0, 64) of a matrix whose rows are `ld` floats apart, in two
// halves so that a block can put the loads of all its tiles in flight before
// it waits for any of them: the groups are small, and with one load
// outstanding per thread the kernel would be bound by memory latency.  Values
// are stored rounded to TF32; rows past `seq` are zero.
template <int HD, int THREADS = kThreads>
struct Staged {
    float4 value[kTile * (HD / 4) / THREADS];
};

template <int HD, int THREADS = kThreads>
__device__ __forceinline__ void stage_load(Staged<HD, THREADS> &staged,
                                           const float *__restrict__ source,
                                           int ld, int seq) {
    constexpr int kVectors = HD / 4;
#pragma unroll
    for (int j = 0; j < kTile * kVectors / THREADS; ++j) {
        const int i = threadIdx.x + j * THREADS;
        const int r = i / kVectors;
        const int c = (i % kVectors) * 4;
        staged.value[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < seq) {
            staged.value[j] = __ldcs(
                reinterpret_cast<const float4 *>(source + size_t(r) * ld + c));
        }
    }
}

template <int HD, int THREADS = kThreads>
__device__ __forceinline__ void stage_store(const Staged<HD, THREADS> &staged,
                                            float *tile) {
    constexpr int kVectors = HD / 4;
#pragma unroll
    for (int j = 0; j < kTile * kVectors / THREADS; ++j) {
        const int i = threadIdx.x + j * THREADS;
        const int r = i / kVectors;
        const int c = (i % kVectors) * 4;
        const float4 v = staged.value[j];
        *reinterpret_cast<float4 *>(tile + tile_index<HD>(r, c)) =
            make_float4(to_tf32(v.x), to_tf32(v.y), to_tf32(v.z), to_tf32(v.w));
    }
}

template <int HD>
__device__ __forceinline__ size_t group_offset(size_t group, int seq,
                                               HeadLayout layout) {
    return (group / layout.heads) * size_t(seq) * layout.ld +
           (group % layout.heads) * HD;
}

// The same for a group index that is a block index: one 32-bit division.
template <int HD>
__device__ __forceinline__ size_t group_offset(unsigned group, int seq,
                                               HeadLayout layout) {
    const unsigned sample = group / unsigned(layout.heads);
    const unsigned head = group - sample * unsigned(layout.heads);
    return size_t(sample) * size_t(unsigned(seq) * unsigned(layout.ld)) +
           head * HD;
}

// ---------------------------------------------------------------------------
// Operands that are not rounded.  mma.sync reads the upper 19 bits of a TF32
// operand register and ignores the rest, so an FP32 value handed over as it is
// gets truncated: a relative error between 0 and 2^-10 that always points
// toward zero.  Its mean (about 0.75 * 2^-11 per operand for mantissas spread
// over [1, 2)) is a bias of every product and is taken out by a constant
// factor on the result, folded into a scale the kernel applies anyway; what
// remains is spread like the error of rounding to nearest.  The kernels for
// whole groups use this to drop every cvt.rna from the instruction stream and
// to stage their tiles with cp.async.
constexpr float kTruncatedOperand = 1.0f + 0.75f / 2048.0f;
constexpr float kTruncatedPair = kTruncatedOperand * kTruncatedOperand;
constexpr float kLog2TruncatedPair = 2.0f * 0.75f / 2048.0f * 1.4426950408889634f;

__device__ __forceinline__ void copy_async_16(float *target, const float *source,
                                              bool valid) {
    const uint32_t address = uint32_t(__cvta_generic_to_shared(target));
    const int bytes = valid ? 16 : 0;   // 0: sixteen zero bytes, nothing is read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
                 :: "r"(address), "l"(source), "r"(bytes) : "memory");
}

__device__ __forceinline__ void copy_async_wait() {
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}

// Rows [0, 32) or [0, 64) of a matrix whose rows are `ld` floats apart (every
// row a 16-row tile that starts below 8 * TILES can touch) go to a staged tile
// as they are, without passing through registers; rows past `seq` become zero.
template <int HD, int TILES>
__device__ __forceinline__ void stage_async(float *tile,
                                            const float *__restrict__ source,
                                            int ld, int seq) {
    constexpr int kVectors = HD / 4;
    constexpr int kRowsPerPass = kThreads / kVectors;   // 8 or 16
    constexpr int kRows = TILES <= 4 ? 32 : kTile;
    const int r = threadIdx.x / kVectors;
    const int c = (threadIdx.x % kVectors) * 4;
    // Both layouts repeat every eight rows.
    float *target = tile + tile_index<HD>(r, c);
    const float *from = source + size_t(r) * ld + c;
#pragma unroll
    for (int j = 0; j < kRows / kRowsPerPass; ++j) {
        const bool valid = r + j * kRowsPerPass < seq;
        copy_async_16(target + j * kRowsPerPass * Shape<HD>::kPitch,
                      valid ? from + size_t(j * kRowsPerPass) * ld : source,
                      valid);
    }
}

// c[16 x 64] += A B^T: A = rows (a0, a1) given as lane ranges, B = a staged
// tile whose rows are the result's columns.
// `live` (< TILES) restricts the work to the first `live` 8-row groups of the
// tile when kPartial is set (the last tile of a streamed axis).
template <int HD, int TILES, bool kPartial = false>
__device__ __forceinline__ void product_rows(float (&c)[8][4],
                                             const float (&a0)[HD / 4],
                                             const float (&a1)[HD / 4],
                                             const float *tile, int g, int t,
                                             int live = TILES) {
    using S = Shape<HD>;
    // Both layouts repeat every eight rows, so the lane's position within a
    // group of eight is computed once and the groups are immediate offsets.
    int lane_chunks[S::kRange / 4];
#pragma unroll
    for (int i = 0; i < S::kRange / 4; ++i) {
        lane_chunks[i] = tile_index<HD>(g, lane_column<HD>(t, 4 * i));
    }
#pragma unroll
    for (int n = 0; n < TILES; ++n) {
        if (!kPartial || n < live) {
            float b[S::kRange];
#pragma unroll
            for (int i = 0; i < S::kRange / 4; ++i) {
                const float4 v = *reinterpret_cast<const float4 *>(
                    tile + n * 8 * S::kPitch + lane_chunks[i]);
                b[4 * i] = v.x; b[4 * i + 1] = v.y;
                b[4 * i + 2] = v.z; b[4 * i + 3] = v.w;
            }
#pragma unroll
            for (int s = 0; s < S::kSteps; ++s) {
                mma_tf32(c[n], a0[2 * s], a1[2 * s], a0[2 * s + 1],
                         a1[2 * s + 1], b[2 * s], b[2 * s + 1]);
            }
        }
    }
}

// o[16 x HD] += P B: P = an accumulator tile set reused as the A operand
// (columns 2t, 2t+1 of tile s), B = a staged tile whose rows are the
// contraction index.  Result element e of the lane's row range is
// o[e % kOut][e / kOut] (row g) and o[e % kOut][2 + e / kOut] (row g + 8).
template <int HD, int TILES, bool kPartial = false, bool kRounded = true>
__device__ __forceinline__ void product_columns(float (&o)[HD / 8][4],
                                                const float (&p)[8][4],
                                                const float *tile, int g,
                                                int t, int live = TILES) {
    using S = Shape<HD>;
    // The lane's 16-byte chunks of rows 2t and 2t + 1 (a swizzled layout does
    // not keep consecutive chunks next to each other).
    constexpr int kChunks = S::kOut < 4 ? 1 : S::kOut / 4;
    int lane_row[kChunks], lane_next[kChunks];
#pragma unroll
    for (int i = 0; i < kChunks; ++i) {
        lane_row[i] = tile_index<HD>(2 * t, g * S::kOut + 4 * i);
        lane_next[i] = tile_index<HD>(2 * t + 1, g * S::kOut + 4 * i);
    }
#pragma unroll
    for (int s = 0; s < TILES; ++s) {
        if (!kPartial || s < live) {
            float b0[S::kOut < 4 ? 4 : S::kOut], b1[S::kOut < 4 ? 4 : S::kOut];
            const float *group = tile + s * 8 * S::kPitch;
            if (S::kOut == 2) {
                const float2 x = *reinterpret_cast<const float2 *>(group + lane_row[0]);
                const float2 y = *reinterpret_cast<const float2 *>(group + lane_next[0]);
                b0[0] = x.x; b0[1] = x.y; b1[0] = y.x; b1[1] = y.y;
            } else {
#pragma unroll
                for (int i = 0; i < S::kOut; i += 4) {
                    const float4 x = *reinterpret_cast<const float4 *>(group + lane_row[i / 4]);
                    const float4 y = *reinterpret_cast<const float4 *>(group + lane_next[i / 4]);
                    b0[i] = x.x; b0[i + 1] = x.y; b0[i + 2] = x.z; b0[i + 3] = x.w;
                    b1[i] = y.x; b1[i + 1] = y.y; b1[i + 2] = y.z; b1[i + 3] = y.w;
                }
            }
            const float a0 = kRounded ? to_tf32(p[s][0]) : p[s][0];
            const float a1 = kRounded ? to_tf32(p[s][2]) : p[s][2];
            const float a2 = kRounded ? to_tf32(p[s][1]) : p[s][1];
            const float a3 = kRounded ? to_tf32(p[s][3]) : p[s][3];
#pragma unroll
            for (int u = 0; u < S::kOut; ++u) {
                mma_tf32(o[u], a0, a1, a2, a3, b0[u], b1[u]);
            }
        }
    }
}

// Writes (or adds) the lane's ranges of result rows r0 and r1.
template <int HD>
__device__ __forceinline__ void store_result(float *base, int ld, int r0, int r1,
                                             int seq, int t,
                                             const float (&o)[HD / 8][4],
                                             bool add) {
    using S = Shape<HD>;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int row = half ? r1 : r0;
        if (row < seq) {
            float *target = base + size_t(row) * ld + t * S::kRange;
#pragma unroll
            for (int e = 0; e < S::kRange; e += 4) {
                float4 v = add ? *reinterpret_cast<float4 *>(target + e)
                               : make_float4(0.f, 0.f, 0.f, 0.f);
                v.x += o[(e + 0) % S::kOut][2 * half + (e + 0) / S::kOut];
                v.y += o[(e + 1) % S::kOut][2 * half + (e + 1) / S::kOut];
                v.z += o[(e + 2) % S::kOut][2 * half + (e + 2) / S::kOut];
                v.w += o[(e + 3) % S::kOut][2 * half + (e + 3) / S::kOut];
                *reinterpret_cast<float4 *>(target + e) = v;
            }
        }
    }
}

// Adds this lane's two rows of a 16 x HD result tile (rows past `seq`
// excluded) to its running column sums, indexed like the lane's row range (see
// store_result); the eight lanes that share the columns are combined once, at
// the end of the kernel.
template <int HD>
__device__ __forceinline__ void add_column_sums(float (&sums)[HD / 4],
                                                const float (&o)[HD / 8][4],
                                                int r0, int r1, int seq) {
    using S = Shape<HD>;
    const float keep0 = r0 < seq ? 1.0f : 0.0f, keep1 = r1 < seq ? 1.0f : 0.0f;
#pragma unroll
    for (int e = 0; e < S::kRange; ++e) {
        sums[e] += keep0 * o[e % S::kOut][e / S::kOut] +
                   keep1 * o[e % S::kOut][2 + e / S::kOut];
    }
}

template <int N>
__device__ __forceinline__ void clear(float (&c)[N][4]) {
#pragma unroll
    for (int n = 0; n < N; ++n) {
        c[n][0] = c[n][1] = c[n][2] = c[n][3] = 0.0f;
    }
}

// Row-wise softmax of a 16 x 64 accumulator tile set holding raw scores, up
// to the normalisation: s becomes exp2(scale2 * (s - max)) with columns >= seq
// at zero; the caller applies 1 / sum where it is cheapest.  Also returns the
// two rows' log-sum-exp (base 2, of the scaled scores).  scale2 > 0.
template <int TILES>
__device__ __forceinline__ void softmax_rows(float (&s)[8][4], int seq, int t,
                                             float scale2, float &inverse_a,
                                             float &inverse_b, float &lse_a,
                                             float &lse_b) {
    float max_a = -FLT_MAX, max_b = -FLT_MAX;
#pragma unroll
    for (int n = 0; n < TILES; ++n) {
        if (n * 8 + 8 > seq) {   // only the tiles that reach past the end
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                if (n * 8 + 2 * t + (e & 1) >= seq) {
                    s[n][e] = -FLT_MAX;
                }
            }
        }
        max_a = fmaxf(max_a, fmaxf(s[n][0], s[n][1]));
        max_b = fmaxf(max_b, fmaxf(s[n][2], s[n][3]));
    }
    max_a = quad_max(max_a);
    max_b = quad_max(max_b);
    const float shift_a = -max_a * scale2, shift_b = -max_b * scale2;
    float sum_a = 0.0f, sum_b = 0.0f;
#pragma unroll
    for (int n = 0; n < TILES; ++n) {
        // A masked entry is -FLT_MAX: the product overflows to -inf, exp2 -> 0.
        s[n][0] = exp2_fast(fmaf(s[n][0], scale2, shift_a));
        s[n][1] = exp2_fast(fmaf(s[n][1], scale2, shift_a));
        s[n][2] = exp2_fast(fmaf(s[n][2], scale2, shift_b));
        s[n][3] = exp2_fast(fmaf(s[n][3], scale2, shift_b));
        sum_a += s[n][0] + s[n][1];
        sum_b += s[n][2] + s[n][3];
    }
    sum_a = quad_sum(sum_a);
    sum_b = quad_sum(sum_b);
    inverse_a = 1.0f / sum_a;
    inverse_b = 1.0f / sum_b;
    lse_a = max_a * scale2 + log2f(sum_a);
    lse_b = max_b * scale2 + log2f(sum_b);
}

template <int HD, int TILES>
__global__ void __launch_bounds__(kThreads, HD == 16 ? 16 : 8)
attention_warp_forward_kernel(const float *__restrict__ q,
                              const float *__restrict__ k,
                              const float *__restrict__ v,
                              float *__restrict__ out, int seq, float scale,
                              HeadLayout in_layout, HeadLayout out_layout) {
    using S = Shape<HD>;
    __shared__ __align__(16) float k_tile[kTile * S::kPitch];
    __shared__ __align__(16) float v_tile[kTile * S::kPitch];
    grid_dependency_wait();
    grid_dependency_release();
    const unsigned group = blockIdx.x;
    const size_t in_base = group_offset<HD>(group, seq, in_layout);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    // All global loads of the block go out together: the K and V tiles
    // (asynchronous copies, unrounded) and the query rows of this warp's (at
    // most two) row tiles.  Rows past the end repeat the last row; their
    // results are dropped.
    stage_async<HD, TILES>(k_tile, k + in_base, in_layout.ld, seq);
    stage_async<HD, TILES>(v_tile, v + in_base, in_layout.ld, seq);
    float query[2][2][S::kRange];
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
        const int r0 = (warp + pass * kWarps) * 16 + g;
        load_range_global(query[pass][0], q + in_base + size_t(min(r0, seq - 1)) * in_layout.ld + t * S::kRange, false);
        load_range_global(query[pass][1], q + in_base + size_t(min(r0 + 8, seq - 1)) * in_layout.ld + t * S::kRange, false);
    }
    copy_async_wait();
    __syncthreads();
    float *out_base = out + group_offset<HD>(group, seq, out_layout);
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
        const int m0 = (warp + pass * kWarps) * 16;
        if (m0 >= seq) {
            break;
        }
        const int r0 = m0 + g, r1 = r0 + 8;
        const float (&a0)[S::kRange] = query[pass][0];
        const float (&a1)[S::kRange] = query[pass][1];
        float p[8][4];
        clear(p);
        product_rows<HD, TILES>(p, a0, a1, k_tile, g, t);
        float inverse_a, inverse_b, lse_a, lse_b;
        softmax_rows<TILES>(p, seq, t, scale * (kLog2e * kTruncatedPair),
                            inverse_a, inverse_b, lse_a, lse_b);
        float o[S::kOut][4];
        clear(o);
        product_columns<HD, TILES, false, false>(o, p, v_tile, g, t);
        // The probabilities were left unnormalised: scale the 16 x HD result
        // instead of the 16 x 64 tile (and undo the truncation of P and V).
        inverse_a *= kTruncatedPair;
        inverse_b *= kTruncatedPair;
#pragma unroll
        for (int u = 0; u < S::kOut; ++u) {
            o[u][0] *= inverse_a;
            o[u][1] *= inverse_a;
            o[u][2] *= inverse_b;
            o[u][3] *= inverse_b;
        }
        store_result<HD>(out_base, out_layout.ld, r0, r1, seq, t, o, false);
    }
}

// Backward.  Pass 1 (query tiles): P, D, dS row-wise, dQ.  Pass 2 (key tiles):
// P^T and dS^T from swapped operands and pass 1's row statistics, dV and dK.
// Register caps: at head dimension 16 the compiler would take 126 registers;
// 112 costs no spill and leaves room next to the eight resident blocks (four
// warps per scheduler either way).  168 is what the 32-wide instantiations use
// anyway.
template <int HD, int TILES>
__global__ void __launch_bounds__(kThreads) __maxnreg__(HD == 16 ? 112 : 168)
attention_warp_backward_kernel(
    const float *__restrict__ q, const float *__restrict__ k,
    const float *__restrict__ v, const float *__restrict__ out,
    const float *__restrict__ dout, float *__restrict__ dq,
    float *__restrict__ dk, float *__restrict__ dv, int seq, float scale,
    bool add_q, bool add_k, bool add_v, HeadLayout in_layout,
    HeadLayout out_layout, HeadLayout dout_layout, HeadLayout grad_layout,
    float *__restrict__ column_partials) {
    using S = Shape<HD>;
    __shared__ __align__(16) float q_tile[kTile * S::kPitch];
    __shared__ __align__(16) float k_tile[kTile * S::kPitch];
    __shared__ __align__(16) float v_tile[kTile * S::kPitch];
    __shared__ __align__(16) float g_tile[kTile * S::kPitch];
    __shared__ __align__(8) float row_lse[kTile];
    __shared__ __align__(8) float row_dot[kTile];
    grid_dependency_wait();
    grid_dependency_release();
    const unsigned group = blockIdx.x;
    const size_t in_base = group_offset<HD>(group, seq, in_layout);
    const float *out_base = out + group_offset<HD>(group, seq, out_layout);
    const float *dout_base = dout + group_offset<HD>(group, seq, dout_layout);
    const size_t grad_base = group_offset<HD>(group, seq, grad_layout);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    // All global loads of the block go out together: the four operand tiles
    // (asynchronous copies, unrounded) and the O rows behind D_i = dO_i . O_i
    // for this warp's (at most two) row tiles; the dO rows of that product
    // are the fragments the first pass reads from the staged tile anyway.
    stage_async<HD, TILES>(q_tile, q + in_base, in_layout.ld, seq);
    stage_async<HD, TILES>(k_tile, k + in_base, in_layout.ld, seq);
    stage_async<HD, TILES>(v_tile, v + in_base, in_layout.ld, seq);
    stage_async<HD, TILES>(g_tile, dout_base, dout_layout.ld, seq);
    float out_rows[2][2][S::kRange];
    float sums[3][S::kRange] = {};   // column sums of dQ, dK, dV (this warp's tiles)
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int row = (warp + pass * kWarps) * 16 + g + 8 * half;
            load_range_global(out_rows[pass][half],
                              out_base + size_t(min(row, seq - 1)) * out_layout.ld + t * S::kRange,
                              false);
        }
    }
    // Rows past the end: P^T must vanish there (lse = +inf) and D is unused.
    for (int i = seq + threadIdx.x; i < kTile; i += kThreads) {
        row_lse[i] = FLT_MAX;
        row_dot[i] = 0.0f;
    }
    copy_async_wait();
    __syncthreads();
    // Every product below has two truncated operands (see kTruncatedPair).
    const float scale2 = scale * (kLog2e * kTruncatedPair);
    const float scale_pair = scale * kTruncatedPair;
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
        const int m0 = (warp + pass * kWarps) * 16;
        if (m0 >= seq) {
            break;
        }
        const int r0 = m0 + g, r1 = r0 + 8;
        float a0[S::kRange], a1[S::kRange];
        load_range(a0, q_tile + tile_index<HD>(r0, t * S::kRange));
        load_range(a1, q_tile + tile_index<HD>(r1, t * S::kRange));
        float p[8][4];
        clear(p);
        product_rows<HD, TILES>(p, a0, a1, k_tile, g, t);
        float inverse_a, inverse_b, lse_a, lse_b;
        softmax_rows<TILES>(p, seq, t, scale2, inverse_a, inverse_b, lse_a,
                            lse_b);
        // dP = dO V^T, then dS = scale P (dP - D) in place over dP.
        load_range(a0, g_tile + tile_index<HD>(r0, t * S::kRange));
        load_range(a1, g_tile + tile_index<HD>(r1, t * S::kRange));
        float dot_a = 0.0f, dot_b = 0.0f;
#pragma unroll
        for (int e = 0; e < S::kRange; ++e) {
            dot_a = fmaf(out_rows[pass][0][e], a0[e], dot_a);
            dot_b = fmaf(out_rows[pass][1][e], a1[e], dot_b);
        }
        dot_a = quad_sum(dot_a);
        dot_b = quad_sum(dot_b);
        if (t == 0) {
            // What the second pass reads: the log-sum-exp lowered so that its
            // P^T comes out scaled for the two products it feeds.
            if (r0 < seq) {
                row_lse[r0] = lse_a - kLog2TruncatedPair;
                row_dot[r0] = -scale * dot_a;
            }
            if (r1 < seq) {
                row_lse[r1] = lse_b - kLog2TruncatedPair;
                row_dot[r1] = -scale * dot_b;
            }
        }
        float ds[8][4];
        clear(ds);
        product_rows<HD, TILES>(ds, a0, a1, v_tile, g, t);
        // p holds exp2(.) without the 1 / sum: fold it into the row factor,
        // with one correction for dP and one for the product dS feeds.
        const float offset_a = -dot_a * scale_pair * inverse_a;
        const float offset_b = -dot_b * scale_pair * inverse_b;
        const float factor_a = scale_pair * kTruncatedPair * inverse_a;
        const float factor_b = scale_pair * kTruncatedPair * inverse_b;
#pragma unroll
        for (int n = 0; n < TILES; ++n) {
            ds[n][0] = p[n][0] * fmaf(ds[n][0], factor_a, offset_a);
            ds[n][1] = p[n][1] * fmaf(ds[n][1], factor_a, offset_a);
            ds[n][2] = p[n][2] * fmaf(ds[n][2], factor_b, offset_b);
            ds[n][3] = p[n][3] * fmaf(ds[n][3], factor_b, offset_b);
        }
        float result[S::kOut][4];
        clear(result);
        product_columns<HD, TILES, false, false>(result, ds, k_tile, g, t);
        store_result<HD>(dq + grad_base, grad_layout.ld, r0, r1, seq, t, result,
                         add_q);
        if (column_partials) {
            add_column_sums<HD>(sums[0], result, r0, r1, seq);
        }
    }
    __syncthreads();
    for (int m0 = warp * 16; m0 < seq; m0 += kWarps * 16) {
        const int r0 = m0 + g, r1 = r0 + 8;   // key rows
        float a0[S::kRange], a1[S::kRange];
        load_range(a0, k_tile + tile_index<HD>(r0, t * S::kRange));
        load_range(a1, k_tile + tile_index<HD>(r1, t * S::kRange));
        float p[8][4];
        clear(p);
        product_rows<HD, TILES>(p, a0, a1, q_tile, g, t);   // S^T
        // Columns are queries here: normalise with their saved statistics.
#pragma unroll
        for (int n = 0; n < TILES; ++n) {
            const float2 lse = *reinterpret_cast<const float2 *>(row_lse + n * 8 + 2 * t);
            p[n][0] = exp2_fast(p[n][0] * scale2 - lse.x);
            p[n][1] = exp2_fast(p[n][1] * scale2 - lse.y);
            p[n][2] = exp2_fast(p[n][2] * scale2 - lse.x);
            p[n][3] = exp2_fast(p[n][3] * scale2 - lse.y);
        }
        float result[S::kOut][4];
        clear(result);
        product_columns<HD, TILES, false, false>(result, p, g_tile, g, t);   // dV = P^T dO
        store_result<HD>(dv + grad_base, grad_layout.ld, r0, r1, seq, t, result,
                         add_v);
        if (column_partials) {
            add_column_sums<HD>(sums[2], result, r0, r1, seq);
        }
        load_range(a0, v_tile + tile_index<HD>(r0, t * S::kRange));
        load_range(a1, v_tile + tile_index<HD>(r1, t * S::kRange));
        float ds[8][4];
        clear(ds);
        product_rows<HD, TILES>(ds, a0, a1, g_tile, g, t);   // dP^T = V dO^T
#pragma unroll
        for (int n = 0; n < TILES; ++n) {
            // row_dot holds -scale * D_i.
            const float2 dot = *reinterpret_cast<const float2 *>(row_dot + n * 8 + 2 * t);
            ds[n][0] = p[n][0] * fmaf(ds[n][0], scale_pair, dot.x);
            ds[n][1] = p[n][1] * fmaf(ds[n][1], scale_pair, dot.y);
            ds[n][2] = p[n][2] * fmaf(ds[n][2], scale_pair, dot.x);
            ds[n][3] = p[n][3] * fmaf(ds[n][3], scale_pair, dot.y);
        }
        clear(result);
        product_columns<HD, TILES, false, false>(result, ds, q_tile, g, t);   // dK = dS^T Q
        store_result<HD>(dk + grad_base, grad_layout.ld, r0, r1, seq, t, result,
                         add_k);
        if (column_partials) {
            add_column_sums<HD>(sums[1], result, r0, r1, seq);
        }
    }
    if (column_partials) {
        // Row `sample` of the partial matrix, in the column order of the
        // projected gradient: [dQ | dK | dV] x heads x HD.  Warp 1 parks its
        // sums in shared memory (the operand tiles are no longer needed),
        // warp 0 adds its own and writes.
#pragma unroll
        for (int which = 0; which < 3; ++which) {
#pragma unroll
            for (int e = 0; e < S::kRange; ++e) {
                float v = sums[which][e];
                v += __shfl_xor_sync(kFullMask, v, 4);
                v += __shfl_xor_sync(kFullMask, v, 8);
                v += __shfl_xor_sync(kFullMask, v, 16);
                sums[which][e] = v;
            }
        }
        __syncthreads();
        float *parked = q_tile;
        if (warp == 1 && g == 0) {
#pragma unroll
            for (int which = 0; which < 3; ++which) {
#pragma unroll
                for (int e = 0; e < S::kRange; ++e) {
                    parked[which * HD + t * S::kRange + e] = sums[which][e];
                }
            }
        }
        __syncthreads();
        if (warp == 0 && g == 0) {
            const int heads = grad_layout.heads;
            const size_t d_model = size_t(heads) * HD;
            float *row = column_partials + (group / heads) * 3 * d_model +
                         (group % heads) * HD + t * S::kRange;
#pragma unroll
            for (int which = 0; which < 3; ++which) {
#pragma unroll
                for (int e = 0; e < S::kRange; e += 4) {
                    float4 v;
                    v.x = sums[which][e + 0] + parked[which * HD + t * S::kRange + e + 0];
                    v.y = sums[which][e + 1] + parked[which * HD + t * S::kRange + e + 1];
                    v.z = sums[which][e + 2] + parked[which * HD + t * S::kRange + e + 2];
                    v.w = sums[which][e + 3] + parked[which * HD + t * S::kRange + e + 3];
                    *reinterpret_cast<float4 *>(row + which * d_model + e) = v;
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Any sequence length: the same register-resident products, streamed over
// 64-row tiles of the other axis (flash attention).  A block of four warps owns
// 64 rows (a warp 16); the tiles it sweeps are staged in shared memory by all
// four warps.  The forward pass keeps a running maximum and denominator per
// row and saves the row's log-sum-exp (base 2, of the scaled scores); the two
// backward kernels rebuild P tiles from it.
//
//   forward        per query tile: for key tiles: S, online softmax, O += P V
//   backward rows  per query tile: D = dO.O (saved, pre-multiplied by -scale);
//                  for key tiles: P, dP = dO V^T, dS, dQ += dS K
//   backward cols  per key tile: for query tiles: P^T = f(K Q^T, lse),
//                  dV += P^T dO, dP^T = V dO^T, dS^T, dK += dS^T Q
constexpr int kStreamWarps = 4;
constexpr int kStreamBlock = kStreamWarps * 32;

// Masks the columns of a 16 x 64 score tile set that lie at or past `limit`
// (columns are counted from the tile's first key).
__device__ __forceinline__ void mask_columns(float (&s)[8][4], int limit, int t) {
#pragma unroll
    for (int n = 0; n < 8; ++n) {
        if (n * 8 + 8 > limit) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                if (n * 8 + 2 * t + (e & 1) >= limit) {
                    s[n][e] = -FLT_MAX;
                }
            }
        }
    }
}

template <int HD>
__device__ __forceinline__ void attention_stream_forward_body(const float *__restrict__ q,
                                const float *__restrict__ k,
                                const float *__restrict__ v,
                                float *__restrict__ out,
                                float *__restrict__ lse, int seq, float scale,
                                HeadLayout in_layout, HeadLayout out_layout) {
    using S = Shape<HD>;
    __shared__ __align__(16) float k_tile[kTile * S::kPitch];
    __shared__ __align__(16) float v_tile[kTile * S::kPitch];
    // Blocks of one group are neighbours in launch order, so that the K / V
    // tiles they all sweep stay in L2.
    const int row_tiles = (seq + kTile - 1) / kTile;
    const size_t group = blockIdx.x / row_tiles;
    const int row_tile = blockIdx.x % row_tiles;
    const size_t base = group_offset<HD>(group, seq, in_layout);
    const int ld = in_layout.ld;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int r0 = row_tile * kTile + warp * 16 + g, r1 = r0 + 8;
    const bool live_warp = row_tile * kTile + warp * 16 < seq;   // else: staging only
    const float scale2 = scale * kLog2e;
    float a0[S::kRange], a1[S::kRange];
    load_lane_global<HD>(a0, q + base + size_t(min(r0, seq - 1)) * ld, t, true);
    load_lane_global<HD>(a1, q + base + size_t(min(r1, seq - 1)) * ld, t, true);
    float max_a = -FLT_MAX, max_b = -FLT_MAX;   // running maxima of raw scores
    float sum_a = 0.0f, sum_b = 0.0f;           // this lane's share of the denominators
    float o[S::kOut][4];
    clear(o);
    for (int k0 = 0; k0 < seq; k0 += kTile) {
        __syncthreads();   // the previous tiles have been consumed
        {
            Staged<HD, kStreamBlock> k_staged, v_staged;
            stage_load<HD, kStreamBlock>(k_staged, k + base + size_t(k0) * ld, ld, seq - k0);
            stage_load<HD, kStreamBlock>(v_staged, v + base + size_t(k0) * ld, ld, seq - k0);
            stage_store<HD, kStreamBlock>(k_staged, k_tile);
            stage_store<HD, kStreamBlock>(v_staged, v_tile);
        }
        __syncthreads();
        if (!live_warp) {
            continue;
        }
        const int live = (min(kTile, seq - k0) + 7) / 8;   // 8-key groups in this tile
        float p[8][4];
        clear(p);
        if (live == 8) {
            product_rows<HD, 8>(p, a0, a1, k_tile, g, t);
        } else {
            product_rows<HD, 8, true>(p, a0, a1, k_tile, g, t, live);
        }
        if (k0 + kTile > seq) {
            mask_columns(p, seq - k0, t);
        }
        float tile_a = -FLT_MAX, tile_b = -FLT_MAX;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            tile_a = fmaxf(tile_a, fmaxf(p[n][0], p[n][1]));
            tile_b = fmaxf(tile_b, fmaxf(p[n][2], p[n][3]));
        }
        const float new_a = fmaxf(max_a, quad_max(tile_a));
        const float new_b = fmaxf(max_b, quad_max(tile_b));
        // Rescale what has been accumulated under the old maximum (the first
        // tile multiplies zeros by exp2(-inf) = 0).
        const float alpha_a = exp2_fast((max_a - new_a) * scale2);
        const float alpha_b = exp2_fast((max_b - new_b) * scale2);
        const float shift_a = -new_a * scale2, shift_b = -new_b * scale2;
        max_a = new_a;
        max_b = new_b;
        float part_a = 0.0f, part_b = 0.0f;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            p[n][0] = exp2_fast(fmaf(p[n][0], scale2, shift_a));
            p[n][1] = exp2_fast(fmaf(p[n][1], scale2, shift_a));
            p[n][2] = exp2_fast(fmaf(p[n][2], scale2, shift_b));
            p[n][3] = exp2_fast(fmaf(p[n][3], scale2, shift_b));
            part_a += p[n][0] + p[n][1];
            part_b += p[n][2] + p[n][3];
        }
        sum_a = fmaf(sum_a, alpha_a, part_a);
        sum_b = fmaf(sum_b, alpha_b, part_b);
#pragma unroll
        for (int u = 0; u < S::kOut; ++u) {
            o[u][0] *= alpha_a;
            o[u][1] *= alpha_a;
            o[u][2] *= alpha_b;
            o[u][3] *= alpha_b;
        }
        if (live == 8) {
            product_columns<HD, 8>(o, p, v_tile, g, t);
        } else {
            product_columns<HD, 8, true>(o, p, v_tile, g, t, live);
        }
    }
    if (!live_warp) {
        return;
    }
    sum_a = quad_sum(sum_a);
    sum_b = quad_sum(sum_b);
    const float inverse_a = 1.0f / sum_a, inverse_b = 1.0f / sum_b;
#pragma unroll
    for (int u = 0; u < S::kOut; ++u) {
        o[u][0] *= inverse_a;
        o[u][1] *= inverse_a;
        o[u][2] *= inverse_b;
        o[u][3] *= inverse_b;
    }
    store_result<HD>(out + group_offset<HD>(group, seq, out_layout),
                     out_layout.ld, r0, r1, seq, t, o, false);
    if (t == 0) {
        if (r0 < seq) {
            lse[group * seq + r0] = max_a * scale2 + log2f(sum_a);
        }
        if (r1 < seq) {
            lse[group * seq + r1] = max_b * scale2 + log2f(sum_b);
        }
    }
}

// Thin entry points: the occupancy target (four blocks per SM, 128 registers)
// pays for head dimensions up to 32 and costs spills at 64.
template <int HD>
__global__ void __launch_bounds__(kStreamBlock)
attention_stream_forward_kernel(const float *__restrict__ q,
                                const float *__restrict__ k,
                                const float *__restrict__ v,
                                float *__restrict__ out,
                                float *__restrict__ lse, int seq, float scale,
                                HeadLayout in_layout, HeadLayout out_layout) {
    attention_stream_forward_body<HD>(q, k, v, out, lse, seq, scale, in_layout, out_layout);
}

template <int HD>
__global__ void __launch_bounds__(kStreamBlock, 4)
attention_stream_forward_dense_kernel(const float *__restrict__ q,
                                const float *__restrict__ k,
                                const float *__restrict__ v,
                                float *__restrict__ out,
                                float *__restrict__ lse, int seq, float scale,
                                HeadLayout in_layout, HeadLayout out_layout) {
    attention_stream_forward_body<HD>(q, k, v, out, lse, seq, scale, in_layout, out_layout);
}

// dQ, and D_i = dO_i . O_i saved as -scale * D_i for the column kernel.
template <int HD>
__device__ __forceinline__ void attention_stream_backward_rows_body(
    const float *__restrict__ q, const float *__restrict__ k,
    const float *__restrict__ v, const float *__restrict__ out,
    const float *__restrict__ dout, const float *__restrict__ lse,
    float *__restrict__ dq, float *__restrict__ row_dots, int seq, float scale,
    bool add_q, HeadLayout in_layout, HeadLayout out_layout,
    HeadLayout dout_layout, HeadLayout grad_layout) {
    using S = Shape<HD>;
    __shared__ __align__(16) float k_tile[kTile * S::kPitch];
    __shared__ __align__(16) float v_tile[kTile * S::kPitch];
    const int row_tiles = (seq + kTile - 1) / kTile;
    const size_t group = blockIdx.x / row_tiles;
    const int row_tile = blockIdx.x % row_tiles;
    const size_t base = group_offset<HD>(group, seq, in_layout);
    const int ld = in_layout.ld;
    const float *out_base = out + group_offset<HD>(group, seq, out_layout);
    const float *dout_base = dout + group_offset<HD>(group, seq, dout_layout);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int r0 = row_tile * kTile + warp * 16 + g, r1 = r0 + 8;
    const bool live_warp = row_tile * kTile + warp * 16 < seq;
    const int safe0 = min(r0, seq - 1), safe1 = min(r1, seq - 1);
    const float scale2 = scale * kLog2e;
    float qa[S::kRange], qb[S::kRange], ga[S::kRange], gb[S::kRange];
    float offset_a, offset_b;   // -scale * D
    {
        float oa[S::kRange], ob[S::kRange];
        load_lane_global<HD>(qa, q + base + size_t(safe0) * ld, t, true);
        load_lane_global<HD>(qb, q + base + size_t(safe1) * ld, t, true);
        load_lane_global<HD>(ga, dout_base + size_t(safe0) * dout_layout.ld, t, false);
        load_lane_global<HD>(gb, dout_base + size_t(safe1) * dout_layout.ld, t, false);
        load_lane_global<HD>(oa, out_base + size_t(safe0) * out_layout.ld, t, false);
        load_lane_global<HD>(ob, out_base + size_t(safe1) * out_layout.ld, t, false);
        float dot_a = 0.0f, dot_b = 0.0f;
#pragma unroll
        for (int e = 0; e < S::kRange; ++e) {
            dot_a = fmaf(oa[e], ga[e], dot_a);
            dot_b = fmaf(ob[e], gb[e], dot_b);
            ga[e] = to_tf32(ga[e]);
            gb[e] = to_tf32(gb[e]);
        }
        offset_a = -scale * quad_sum(dot_a);
        offset_b = -scale * quad_sum(dot_b);
        if (t == 0) {
            if (r0 < seq) {
                row_dots[group * seq + r0] = offset_a;
            }
            if (r1 < seq) {
                row_dots[group * seq + r1] = offset_b;
            }
        }
    }
    const float lse_a = lse[group * seq + safe0], lse_b = lse[group * seq + safe1];
    float result[S::kOut][4];
    clear(result);
    for (int k0 = 0; k0 < seq; k0 += kTile) {
        __syncthreads();
        {
            Staged<HD, kStreamBlock> k_staged, v_staged;
            stage_load<HD, kStreamBlock>(k_staged, k + base + size_t(k0) * ld, ld, seq - k0);
            stage_load<HD, kStreamBlock>(v_staged, v + base + size_t(k0) * ld, ld, seq - k0);
            stage_store<HD, kStreamBlock>(k_staged, k_tile);
            stage_store<HD, kStreamBlock>(v_staged, v_tile);
        }
        __syncthreads();
        if (!live_warp) {
            continue;
        }
        const int live = (min(kTile, seq - k0) + 7) / 8;
        float p[8][4];
        float ds[8][4];
        clear(p);
        clear(ds);
        if (live == 8) {
            product_rows<HD, 8>(p, qa, qb, k_tile, g, t);
            product_rows<HD, 8>(ds, ga, gb, v_tile, g, t);
        } else {
            product_rows<HD, 8, true>(p, qa, qb, k_tile, g, t, live);
            product_rows<HD, 8, true>(ds, ga, gb, v_tile, g, t, live);
        }
        if (k0 + kTile > seq) {
            mask_columns(p, seq - k0, t);   // -FLT_MAX: exp2 gives 0 below
        }
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            ds[n][0] = exp2_fast(fmaf(p[n][0], scale2, -lse_a)) * fmaf(ds[n][0], scale, offset_a);
            ds[n][1] = exp2_fast(fmaf(p[n][1], scale2, -lse_a)) * fmaf(ds[n][1], scale, offset_a);
            ds[n][2] = exp2_fast(fmaf(p[n][2], scale2, -lse_b)) * fmaf(ds[n][2], scale, offset_b);
            ds[n][3] = exp2_fast(fmaf(p[n][3], scale2, -lse_b)) * fmaf(ds[n][3], scale, offset_b);
        }
        if (live == 8) {
            product_columns<HD, 8>(result, ds, k_tile, g, t);
        } else {
            product_columns<HD, 8, true>(result, ds, k_tile, g, t, live);
        }
    }
    if (!live_warp) {
        return;
    }
    store_result<HD>(dq + group_offset<HD>(group, seq, grad_layout),
                     grad_layout.ld, r0, r1, seq, t, result, add_q);
}

// Thin entry points: the occupancy target (four blocks per SM, 128 registers)
// pays for head dimensions up to 32 and costs spills at 64.
template <int HD>
__global__ void __launch_bounds__(kStreamBlock)
attention_stream_backward_rows_kernel(
    const float *__restrict__ q, const float *__restrict__ k,
    const float *__restrict__ v, const float *__restrict__ out,
    const float *__restrict__ dout, const float *__restrict__ lse,
    float *__restrict__ dq, float *__restrict__ row_dots, int seq, float scale,
    bool add_q, HeadLayout in_layout, HeadLayout out_layout,
    HeadLayout dout_layout, HeadLayout grad_layout) {
    attention_stream_backward_rows_body<HD>(q, k, v, out, dout, lse, dq, row_dots, seq, scale, add_q, in_layout, out_layout, dout_layout, grad_layout);
}

template <int HD>
__global__ void __launch_bounds__(kStreamBlock, 4)
attention_stream_backward_rows_dense_kernel(
    const float *__restrict__ q, const float *__restrict__ k,
    const float *__restrict__ v, const float *__restrict__ out,
    const float *__restrict__ dout, const float *__restrict__ lse,
    float *__restrict__ dq, float *__restrict__ row_dots, int seq, float scale,
    bool add_q, HeadLayout in_layout, HeadLayout out_layout,
    HeadLayout dout_layout, HeadLayout grad_layout) {
    attention_stream_backward_rows_body<HD>(q, k, v, out, dout, lse, dq, row_dots, seq, scale, add_q, in_layout, out_layout, dout_layout, grad_layout);
}

// dK and dV for a tile of keys, sweeping the queries.
template <int HD>
__device__ __forceinline__ void attention_stream_backward_columns_body(
    const float *__restrict__ q, const float *__restrict__ k,
    const float *__restrict__ v, const float *__restrict__ dout,
    const float *__restrict__ lse, const float *__restrict__ row_dots,
    float *__restrict__ dk, float *__restrict__ dv, int seq, float scale,
    bool add_k, bool add_v, HeadLayout in_layout, HeadLayout dout_layout,
    HeadLayout grad_layout) {
    using S = Shape<HD>;
    __shared__ __align__(16) float q_tile[kTile * S::kPitch];
    __shared__ __align__(16) float g_tile[kTile * S::kPitch];
    __shared__ __align__(8) float tile_lse[kTile];
    __shared__ __align__(8) float tile_dot[kTile];
    const int row_tiles = (seq + kTile - 1) / kTile;
    const size_t group = blockIdx.x / row_tiles;
    const int row_tile = blockIdx.x % row_tiles;
    const size_t base = group_offset<HD>(group, seq, in_layout);
    const int ld = in_layout.ld;
    const float *dout_base = dout + group_offset<HD>(group, seq, dout_layout);
    const size_t grad_base = group_offset<HD>(group, seq, grad_layout);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int r0 = row_tile * kTile + warp * 16 + g, r1 = r0 + 8;   // keys
    const bool live_warp = row_tile * kTile + warp * 16 < seq;
    const int safe0 = min(r0, seq - 1), safe1 = min(r1, seq - 1);
    const float scale2 = scale * kLog2e;
    float ka[S::kRange], kb[S::kRange], va[S::kRange], vb[S::kRange];
    load_lane_global<HD>(ka, k + base + size_t(safe0) * ld, t, true);
    load_lane_global<HD>(kb, k + base + size_t(safe1) * ld, t, true);
    load_lane_global<HD>(va, v + base + size_t(safe0) * ld, t, true);
    load_lane_global<HD>(vb, v + base + size_t(safe1) * ld, t, true);
    float dk_acc[S::kOut][4], dv_acc[S::kOut][4];
    clear(dk_acc);
    clear(dv_acc);
    for (int q0 = 0; q0 < seq; q0 += kTile) {
        __syncthreads();
        {
            Staged<HD, kStreamBlock> q_staged, g_staged;
            stage_load<HD, kStreamBlock>(q_staged, q + base + size_t(q0) * ld, ld, seq - q0);
            stage_load<HD, kStreamBlock>(g_staged, dout_base + size_t(q0) * dout_layout.ld,
                                         dout_layout.ld, seq - q0);
            if (threadIdx.x < kTile) {
                // Queries past the end: an infinite log-sum-exp makes their
                // column of P^T vanish.
                const int row = q0 + threadIdx.x;
                tile_lse[threadIdx.x] = row < seq ? lse[group * seq + row] : FLT_MAX;
                tile_dot[threadIdx.x] = row < seq ? row_dots[group * seq + row] : 0.0f;
            }
            stage_store<HD, kStreamBlock>(q_staged, q_tile);
            stage_store<HD, kStreamBlock>(g_staged, g_tile);
        }
        __syncthreads();
        if (!live_warp) {
            continue;
        }
        const int live = (min(kTile, seq - q0) + 7) / 8;   // 8-query groups
        float p[8][4];
        clear(p);
        if (live == 8) {
            product_rows<HD, 8>(p, ka, kb, q_tile, g, t);   // S^T
        } else {
            product_rows<HD, 8, true>(p, ka, kb, q_tile, g, t, live);
        }
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            const float2 l = *reinterpret_cast<const float2 *>(tile_lse + n * 8 + 2 * t);
            p[n][0] = exp2_fast(fmaf(p[n][0], scale2, -l.x));
            p[n][1] = exp2_fast(fmaf(p[n][1], scale2, -l.y));
            p[n][2] = exp2_fast(fmaf(p[n][2], scale2, -l.x));
            p[n][3] = exp2_fast(fmaf(p[n][3], scale2, -l.y));
        }
        float ds[8][4];
        clear(ds);
        if (live == 8) {
            product_columns<HD, 8>(dv_acc, p, g_tile, g, t);   // dV += P^T dO
            product_rows<HD, 8>(ds, va, vb, g_tile, g, t);     // dP^T = V dO^T
        } else {
            product_columns<HD, 8, true>(dv_acc, p, g_tile, g, t, live);
            product_rows<HD, 8, true>(ds, va, vb, g_tile, g, t, live);
        }
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            const float2 d = *reinterpret_cast<const float2 *>(tile_dot + n * 8 + 2 * t);
            ds[n][0] = p[n][0] * fmaf(ds[n][0], scale, d.x);
            ds[n][1] = p[n][1] * fmaf(ds[n][1], scale, d.y);
            ds[n][2] = p[n][2] * fmaf(ds[n][2], scale, d.x);
            ds[n][3] = p[n][3] * fmaf(ds[n][3], scale, d.y);
        }
        if (live == 8) {
            product_columns<HD, 8>(dk_acc, ds, q_tile, g, t);   // dK += dS^T Q
        } else {
            product_columns<HD, 8, true>(dk_acc, ds, q_tile, g, t, live);
        }
    }
    if (!live_warp) {
        return;
    }
    store_result<HD>(dv + grad_base, grad_layout.ld, r0, r1, seq, t, dv_acc, add_v);
    store_result<HD>(dk + grad_base, grad_layout.ld, r0, r1, seq, t, dk_acc, add_k);
}

// Thin entry points: the occupancy target (four blocks per SM, 128 registers)
// pays for head dimensions up to 32 and costs spills at 64.
template <int HD>
__global__ void __launch_bounds__(kStreamBlock)
attention_stream_backward_columns_kernel(
    const float *__restrict__ q, const float *__restrict__ k,
    const float *__restrict__ v, const float *__restrict__ dout,
    const float *__restrict__ lse, const float *__restrict__ row_dots,
    float *__restrict__ dk, float *__restrict__ dv, int seq, float scale,
    bool add_k, bool add_v, HeadLayout in_layout, HeadLayout dout_layout,
    HeadLayout grad_layout) {
    attention_stream_backward_columns_body<HD>(q, k, v, dout, lse, row_dots, dk, dv, seq, scale, add_k, add_v, in_layout, dout_layout, grad_layout);
}

template <int HD>
__global__ void __launch_bounds__(kStreamBlock, 4)
attention_stream_backward_columns_dense_kernel(
    const float *__restrict__ q, const float *__restrict__ k,
    const float *__restrict__ v, const float *__restrict__ dout,
    const float *__restrict__ lse, const float *__restrict__ row_dots,
    float *__restrict__ dk, float *__restrict__ dv, int seq, float scale,
    bool add_k, bool add_v, HeadLayout in_layout, HeadLayout dout_layout,
    HeadLayout grad_layout) {
    attention_stream_backward_columns_body<HD>(q, k, v, dout, lse, row_dots, dk, dv, seq, scale, add_k, add_v, in_layout, dout_layout, grad_layout);
}

HeadLayout resolve(HeadLayout layout, size_t head_dim) {
    return layout.ld ? layout : HeadLayout{int(head_dim), 1};
}

}  // namespace

// The number of 8-key tiles is a compile-time constant so that the fragment
// loads of a product can all be scheduled ahead of its mma instructions: the
// smallest of 4, 7 (covers the 50-token models) and 8 that holds the sequence.
#define VITB200_WARP_DISPATCH(head_dim, seq, CALL)                             \
    do {                                                                       \
        const int tiles_ = int((seq + 7) / 8);                                 \
        if (head_dim == 16) {                                                  \
            if (tiles_ <= 4) { CALL(16, 4); }                                  \
            else if (tiles_ <= 7) { CALL(16, 7); }                             \
            else { CALL(16, 8); }                                              \
        } else {                                                               \
            if (tiles_ <= 4) { CALL(32, 4); }                                  \
            else if (tiles_ <= 7) { CALL(32, 7); }                             \
            else { CALL(32, 8); }                                              \
        }                                                                      \
    } while (0)

int attention_tile_index(int head_dim, int row, int col) {
    switch (head_dim) {
        case 16: return tile_index<16>(row, col);
        case 32: return tile_index<32>(row, col);
        case 64: return tile_index<64>(row, col);
        default: return -1;
    }
}

int attention_lane_column(int head_dim, int t, int e) {
    switch (head_dim) {
        case 16: return lane_column<16>(t, e);
        case 32: return lane_column<32>(t, e);
        case 64: return lane_column<64>(t, e);
        default: return -1;
    }
}

bool attention_warp_supported(size_t seq, size_t head_dim) {
    return seq >= 1 && seq <= size_t(kTile) && (head_dim == 16 || head_dim == 32);
}

bool launch_attention_warp_forward(const float *q, const float *k,
                                   const float *v, float *out, size_t groups,
                                   size_t seq, size_t head_dim, float scale,
                                   cudaStream_t stream, HeadLayout in_layout,
                                   HeadLayout out_layout) {
    if (!attention_warp_supported(seq, head_dim)) {
        return false;
    }
    in_layout = resolve(in_layout, head_dim);
    out_layout = resolve(out_layout, head_dim);
#define FORWARD(HD, TILES)                                                     \
    launch_chained(attention_warp_forward_kernel<HD, TILES>, unsigned(groups), \
                   kThreads, 0, stream, q, k, v, out, int(seq), scale,         \
                   in_layout, out_layout)
    VITB200_WARP_DISPATCH(head_dim, seq, FORWARD);
#undef FORWARD
    ++g_kernel_launches;
    return true;
}

bool launch_attention_warp_backward(const float *q, const float *k,
                                    const float *v, const float *out,
                                    const float *dout, float *dq, float *dk,
                                    float *dv, size_t groups, size_t seq,
                                    size_t head_dim, float scale, bool add_q,
                                    bool add_k, bool add_v, cudaStream_t stream,
                                    HeadLayout in_layout, HeadLayout out_layout,
                                    HeadLayout dout_layout,
                                    HeadLayout grad_layout,
                                    float *column_partials) {
    if (!attention_warp_supported(seq, head_dim)) {
        return false;
    }
    in_layout = resolve(in_layout, head_dim);
    out_layout = resolve(out_layout, head_dim);
    dout_layout = resolve(dout_layout, head_dim);
    grad_layout = resolve(grad_layout, head_dim);
#define BACKWARD(HD, TILES)                                                    \
    launch_chained(attention_warp_backward_kernel<HD, TILES>, unsigned(groups),\
                   kThreads, 0, stream, q, k, v, out, dout, dq, dk, dv,        \
                   int(seq), scale, add_q, add_k, add_v, in_layout, out_layout,\
                   dout_layout, grad_layout, column_partials)
    VITB200_WARP_DISPATCH(head_dim, seq, BACKWARD);
#undef BACKWARD
    ++g_kernel_launches;
    return true;
}

bool attention_stream_supported(size_t head_dim) {
    return head_dim == 16 || head_dim == 32 || head_dim == 64;
}

#define VITB200_STREAM_DISPATCH(head_dim, CALL)                                \
    do {                                                                       \
        if (head_dim == 16) { CALL(16, _dense_kernel); }                       \
        else if (head_dim == 32) { CALL(32, _dense_kernel); }                  \
        else { CALL(64, _kernel); }                                            \
    } while (0)

bool launch_attention_stream_forward(const float *q, const float *k,
                                     const float *v, float *out, float *lse,
                                     size_t groups, size_t seq, size_t head_dim,
                                     float scale, cudaStream_t stream,
                                     HeadLayout in_layout,
                                     HeadLayout out_layout) {
    if (!attention_stream_supported(head_dim) || seq == 0) {
        return false;
    }
    in_layout = resolve(in_layout, head_dim);
    out_layout = resolve(out_layout, head_dim);
    const unsigned grid = unsigned(groups * ((seq + kTile - 1) / kTile));
#define FORWARD(HD, KIND)                                                      \
    attention_stream_forward##KIND<HD><<<grid, kStreamBlock, 0, stream>>>(     \
        q, k, v, out, lse, int(seq), scale, in_layout, out_layout)
    VITB200_STREAM_DISPATCH(head_dim, FORWARD);
#undef FORWARD
    ++g_kernel_launches;
    return true;
}

bool launch_attention_stream_backward(const float *q, const float *k,
                                      const float *v, const float *out,
                                      const float *dout, const float *lse,
                                      float *dq, float *dk, float *dv,
                                      float *row_dots, size_t groups, size_t seq,
                                      size_t head_dim, float scale, bool add_q,
                                      bool add_k, bool add_v,
                                      cudaStream_t stream, HeadLayout in_layout,
                                      HeadLayout out_layout,
                                      HeadLayout dout_layout,
                                      HeadLayout grad_layout) {
    if (!attention_stream_supported(head_dim) || seq == 0) {
        return false;
    }
    in_layout = resolve(in_layout, head_dim);
    out_layout = resolve(out_layout, head_dim);
    dout_layout = resolve(dout_layout, head_dim);
    grad_layout = resolve(grad_layout, head_dim);
    const unsigned grid = unsigned(groups * ((seq + kTile - 1) / kTile));
#define BACKWARD(HD, KIND)                                                     \
    attention_stream_backward_rows##KIND<HD>                                   \
        <<<grid, kStreamBlock, 0, stream>>>(                                   \
            q, k, v, out, dout, lse, dq, row_dots, int(seq), scale, add_q,     \
            in_layout, out_layout, dout_layout, grad_layout);                  \
    attention_stream_backward_columns##KIND<HD>                                \
        <<<grid, kStreamBlock, 0, stream>>>(                                   \
            q, k, v, dout, lse, row_dots, dk, dv, int(seq), scale, add_k,      \
            add_v, in_layout, dout_layout, grad_layout)
    VITB200_STREAM_DISPATCH(head_dim, BACKWARD);
#undef BACKWARD
    g_kernel_launches += 2;
    return true;
}

}  // namespace vitb200
