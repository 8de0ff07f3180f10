// Attention for short sequences (seq <= 128): one block per (sample, head)
// group with the whole group resident in shared memory, one thread per row.
//
// With 50 tokens and 16-wide heads a group is 9.6 KB of Q/K/V and a 10 KB
// probability matrix, so everything is read from HBM once, the scores never
// leave the SM before they are normalised, and P is written back with fully
// coalesced stores (the host keeps P as a tensor; reference
// src/ops.c:1297-1355).  K and V rows are read by all threads at the same
// address (shared-memory broadcast); each thread's own P row has an odd pitch,
// so row-wise and column-wise walks are both conflict-free.
//
// Backward (reference src/ops.c:1381-1441), three phases on the same tiles:
//   columns  dV_j  = sum_i P_ij dO_i
//   rows     dS_ij = scale P_ij (dO_i.V_j - dO_i.O_i), in place over P;
//            dQ_i  = sum_j dS_ij K_j
//   columns  dK_j  = sum_i dS_ij Q_i
#include "kernels.h"
#include "device_util.cuh"

#include <cfloat>

namespace vitb200 {
namespace {

// Cooperative copy of a [rows, HD] block whose rows are `ld` floats apart into
// a dense shared-memory tile.
template <int HD>
__device__ __forceinline__ void load_rows(const float *__restrict__ source,
                                          float *tile, int rows, int ld) {
    constexpr int kPerRow = HD / 4;
    const int vectors = rows * kPerRow;
    float4 *to = reinterpret_cast<float4 *>(tile);
    for (int i = threadIdx.x; i < vectors; i += blockDim.x) {
        const int row = i / kPerRow, chunk = i % kPerRow;
        to[i] = __ldcs(reinterpret_cast<const float4 *>(source + size_t(row) * ld) + chunk);
    }
}

// Offset of a group's first row under a layout (see HeadLayout).
template <int HD>
__device__ __forceinline__ size_t group_offset(size_t group, int seq,
                                               HeadLayout layout) {
    return (group / layout.heads) * size_t(seq) * layout.ld +
           (group % layout.heads) * HD;
}

// Packed FP32 arithmetic: Blackwell issues two FP32 FMAs per instruction on
// register pairs (fma.rn.f32x2), which halves the instruction count of the
// short dot products and row updates below.  Rows live in registers as HD/2
// packed pairs.
typedef unsigned long long pair_t;

__device__ __forceinline__ pair_t pack(float lo, float hi) {
    pair_t p;
    asm("mov.b64 %0, {%1, %2};" : "=l"(p) : "f"(lo), "f"(hi));
    return p;
}

__device__ __forceinline__ void unpack(pair_t p, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(p));
}

__device__ __forceinline__ pair_t fma2(pair_t a, pair_t b, pair_t c) {
    pair_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

// row . tile_row; the tile row is read with 128-bit shared-memory loads (every
// thread of the warp reads the same address: one broadcast per load).
template <int HD>
__device__ __forceinline__ float dot_tile(const pair_t (&row)[HD / 2],
                                          const float *tile_row) {
    const float4 *t = reinterpret_cast<const float4 *>(tile_row);
    pair_t sum = pack(0.0f, 0.0f);
#pragma unroll
    for (int c = 0; c < HD / 4; ++c) {
        const float4 x = t[c];
        sum = fma2(row[2 * c], pack(x.x, x.y), sum);
        sum = fma2(row[2 * c + 1], pack(x.z, x.w), sum);
    }
    float lo, hi;
    unpack(sum, lo, hi);
    return lo + hi;
}

// row += a * tile_row.
template <int HD>
__device__ __forceinline__ void axpy_tile(pair_t (&row)[HD / 2], float a,
                                          const float *tile_row) {
    const float4 *t = reinterpret_cast<const float4 *>(tile_row);
    const pair_t a2 = pack(a, a);
#pragma unroll
    for (int c = 0; c < HD / 4; ++c) {
        const float4 x = t[c];
        row[2 * c] = fma2(a2, pack(x.x, x.y), row[2 * c]);
        row[2 * c + 1] = fma2(a2, pack(x.z, x.w), row[2 * c + 1]);
    }
}

template <int HD>
__device__ __forceinline__ void clear_row(pair_t (&row)[HD / 2]) {
#pragma unroll
    for (int c = 0; c < HD / 2; ++c) {
        row[c] = pack(0.0f, 0.0f);
    }
}

// Loads a row of HD floats (global or shared) into packed registers.
template <int HD>
__device__ __forceinline__ void load_row_pairs(pair_t (&row)[HD / 2],
                                               const float *source) {
    const float4 *t = reinterpret_cast<const float4 *>(source);
#pragma unroll
    for (int c = 0; c < HD / 4; ++c) {
        const float4 x = t[c];
        row[2 * c] = pack(x.x, x.y);
        row[2 * c + 1] = pack(x.z, x.w);
    }
}

// target (+)= row, 128-bit global accesses.
template <int HD>
__device__ __forceinline__ void store_row_pairs(float *target,
                                                const pair_t (&row)[HD / 2],
                                                bool add) {
#pragma unroll
    for (int c = 0; c < HD / 4; ++c) {
        float4 *t = reinterpret_cast<float4 *>(target) + c;
        float4 value = add ? *t : make_float4(0.f, 0.f, 0.f, 0.f);
        float a, b, d, e;
        unpack(row[2 * c], a, b);
        unpack(row[2 * c + 1], d, e);
        value.x += a; value.y += b; value.z += d; value.w += e;
        *t = value;
    }
}

// exp for softmax arguments (<= 0 after subtracting the row maximum):
// ex2.approx on x * log2(e), relative error about 2e-7 in this range.
__device__ __forceinline__ float softmax_exp(float x) {
    return __expf(x);
}

// Copies the group's [seq, seq] probability block between global memory
// (contiguous rows) and the padded shared tile, one row per warp at a time.
template <bool kToGlobal>
__device__ __forceinline__ void move_probabilities(float *global_block,
                                                   float *tile, int seq,
                                                   int pitch) {
    const int lane = threadIdx.x & 31;
    const int warps = blockDim.x >> 5;
    for (int r = threadIdx.x >> 5; r < seq; r += warps) {
        for (int c = lane; c < seq; c += 32) {
            if (kToGlobal) {
                global_block[r * seq + c] = tile[r * pitch + c];
            } else {
                tile[r * pitch + c] = __ldcs(global_block + r * seq + c);
            }
        }
    }
}

template <int HD>
__global__ void attention_small_forward_kernel(
    const float *__restrict__ q, const float *__restrict__ k,
    const float *__restrict__ v, float *__restrict__ p, float *__restrict__ out,
    int seq, float scale, bool write_p, bool write_o, HeadLayout in_layout,
    HeadLayout out_layout) {
    extern __shared__ __align__(16) float shared[];
    const int pitch = seq | 1;
    float *k_tile = shared;
    float *v_tile = k_tile + seq * HD;
    float *p_tile = v_tile + seq * HD;
    const size_t group = blockIdx.x;
    const size_t base = group_offset<HD>(group, seq, in_layout);
    load_rows<HD>(k + base, k_tile, seq, in_layout.ld);
    load_rows<HD>(v + base, v_tile, seq, in_layout.ld);
    const int row = threadIdx.x;
    pair_t query[HD / 2];
    if (row < seq) {
        load_row_pairs<HD>(query, q + base + size_t(row) * in_layout.ld);
    }
    __syncthreads();
    if (row < seq) {
        float *scores = p_tile + row * pitch;
        float maximum = -FLT_MAX;
        for (int j = 0; j < seq; ++j) {
            const float dot = scale * dot_tile<HD>(query, k_tile + j * HD);
            scores[j] = dot;
            maximum = fmaxf(maximum, dot);
        }
        float denominator = 0.0f;
        for (int j = 0; j < seq; ++j) {
            const float e = softmax_exp(scores[j] - maximum);
            scores[j] = e;
            denominator += e;
        }
        const float inverse = 1.0f / denominator;
        pair_t result[HD / 2];
        clear_row<HD>(result);
        for (int j = 0; j < seq; ++j) {
            const float probability = scores[j] * inverse;
            scores[j] = probability;
            axpy_tile<HD>(result, probability, v_tile + j * HD);
        }
        if (write_o) {
            store_row_pairs<HD>(out + group_offset<HD>(group, seq, out_layout) +
                                    size_t(row) * out_layout.ld,
                                result, false);
        }
    }
    if (write_p) {
        __syncthreads();
        move_probabilities<true>(p + group * seq * seq, p_tile, seq, pitch);
    }
}

template <int HD>
__global__ void attention_small_backward_kernel(
    const float *__restrict__ q, const float *__restrict__ k,
    const float *__restrict__ v, const float *__restrict__ p,
    const float *__restrict__ out, const float *__restrict__ dout,
    float *__restrict__ dq, float *__restrict__ dk, float *__restrict__ dv,
    int seq, float scale, bool add_q, bool add_k, bool add_v, bool recompute,
    HeadLayout in_layout, HeadLayout out_layout, HeadLayout dout_layout,
    HeadLayout grad_layout) {
    extern __shared__ __align__(16) float shared[];
    const int pitch = seq | 1;
    float *q_tile = shared;
    float *k_tile = q_tile + seq * HD;
    float *v_tile = k_tile + seq * HD;
    float *do_tile = v_tile + seq * HD;
    float *p_tile = do_tile + seq * HD;
    const size_t group = blockIdx.x;
    const size_t base = group_offset<HD>(group, seq, in_layout);
    load_rows<HD>(q + base, q_tile, seq, in_layout.ld);
    load_rows<HD>(k + base, k_tile, seq, in_layout.ld);
    load_rows<HD>(v + base, v_tile, seq, in_layout.ld);
    load_rows<HD>(dout + group_offset<HD>(group, seq, dout_layout), do_tile,
                  seq, dout_layout.ld);
    if (!recompute) {
        move_probabilities<false>(const_cast<float *>(p) + group * seq * seq,
                                  p_tile, seq, pitch);
    }
    const int row = threadIdx.x;
    float row_dot = 0.0f;
    if (row < seq) {
        const float *out_row = out + group_offset<HD>(group, seq, out_layout) +
                               size_t(row) * out_layout.ld;
        const float *dout_row = dout +
                                group_offset<HD>(group, seq, dout_layout) +
                                size_t(row) * dout_layout.ld;
#pragma unroll
        for (int d = 0; d < HD; d += 4) {
            const float4 o =
                __ldcs(reinterpret_cast<const float4 *>(out_row + d));
            const float4 g =
                __ldcs(reinterpret_cast<const float4 *>(dout_row + d));
            row_dot += (o.x * g.x + o.y * g.y) + (o.z * g.z + o.w * g.w);
        }
    }
    __syncthreads();
    if (recompute) {
        // The forward pass did not store P: rebuild this row of it from Q and
        // K with the forward kernel's arithmetic (same order, same rounding).
        if (row < seq) {
            pair_t query[HD / 2];
            load_row_pairs<HD>(query, q_tile + row * HD);
            float *scores = p_tile + row * pitch;
            float maximum = -FLT_MAX;
            for (int j = 0; j < seq; ++j) {
                const float dot = scale * dot_tile<HD>(query, k_tile + j * HD);
                scores[j] = dot;
                maximum = fmaxf(maximum, dot);
            }
            float denominator = 0.0f;
            for (int j = 0; j < seq; ++j) {
                const float e = softmax_exp(scores[j] - maximum);
                scores[j] = e;
                denominator += e;
            }
            const float inverse = 1.0f / denominator;
            for (int j = 0; j < seq; ++j) {
                scores[j] *= inverse;
            }
        }
        __syncthreads();
    }
    pair_t acc[HD / 2];
    const size_t grad_row = group_offset<HD>(group, seq, grad_layout) +
                            size_t(row) * grad_layout.ld;
    // Columns: dV_j = sum_i P_ij dO_i.
    if (row < seq) {
        clear_row<HD>(acc);
        for (int i = 0; i < seq; ++i) {
            axpy_tile<HD>(acc, p_tile[i * pitch + row], do_tile + i * HD);
        }
        store_row_pairs<HD>(dv + grad_row, acc, add_v);
    }
    __syncthreads();
    // Rows: score gradients in place over P, then dQ_i.
    if (row < seq) {
        pair_t g[HD / 2];
        load_row_pairs<HD>(g, do_tile + row * HD);
        clear_row<HD>(acc);
        float *scores = p_tile + row * pitch;
        for (int j = 0; j < seq; ++j) {
            const float dp = dot_tile<HD>(g, v_tile + j * HD);
            const float ds = scale * scores[j] * (dp - row_dot);
            scores[j] = ds;
            axpy_tile<HD>(acc, ds, k_tile + j * HD);
        }
        store_row_pairs<HD>(dq + grad_row, acc, add_q);
    }
    __syncthreads();
    // Columns: dK_j = sum_i dS_ij Q_i.
    if (row < seq) {
        clear_row<HD>(acc);
        for (int i = 0; i < seq; ++i) {
            axpy_tile<HD>(acc, p_tile[i * pitch + row], q_tile + i * HD);
        }
        store_row_pairs<HD>(dk + grad_row, acc, add_k);
    }
}

template <typename Kernel>
bool fit_shared(Kernel kernel, size_t bytes) {
    if (bytes > 200 * 1024) {
        return false;
    }
    if (bytes > 48 * 1024) {
        return cudaFuncSetAttribute(kernel,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    int(bytes)) == cudaSuccess;
    }
    return true;
}

// {0, x} stands for "stored group by group".
HeadLayout resolve_layout(HeadLayout layout, size_t head_dim) {
    return layout.ld ? layout : HeadLayout{int(head_dim), 1};
}

}  // namespace

bool attention_small_supported(size_t seq, size_t head_dim) {
    return seq <= 128 &&
           (head_dim == 8 || head_dim == 16 || head_dim == 32 || head_dim == 64);
}

#define VITB200_DISPATCH_HD(head_dim, CALL)                                    \
    switch (head_dim) {                                                        \
        case 8: CALL(8); break;                                                \
        case 16: CALL(16); break;                                              \
        case 32: CALL(32); break;                                              \
        default: CALL(64); break;                                              \
    }

bool launch_attention_small_forward(const float *q, const float *k,
                                    const float *v, float *probabilities,
                                    float *out, size_t groups, size_t seq,
                                    size_t head_dim, float scale, bool write_p,
                                    bool write_o, cudaStream_t stream,
                                    HeadLayout in_layout,
                                    HeadLayout out_layout) {
    in_layout = resolve_layout(in_layout, head_dim);
    out_layout = resolve_layout(out_layout, head_dim);
    const unsigned threads = unsigned((seq + 31) / 32 * 32);
    const size_t bytes = (2 * seq * head_dim + seq * (seq | 1)) * sizeof(float);
    bool launched = false;
#define CALL(HD)                                                               \
    if (fit_shared(attention_small_forward_kernel<HD>, bytes)) {               \
        attention_small_forward_kernel<HD>                                     \
            <<<unsigned(groups), threads, bytes, stream>>>(                    \
                q, k, v, probabilities, out, int(seq), scale, write_p,         \
                write_o, in_layout, out_layout);                               \
        launched = true;                                                       \
    }
    VITB200_DISPATCH_HD(head_dim, CALL)
#undef CALL
    g_kernel_launches += launched ? 1 : 0;
    return launched;
}

bool launch_attention_small_backward(const float *q, const float *k,
                                     const float *v, const float *probabilities,
                                     const float *out, const float *dout,
                                     float *dq, float *dk, float *dv,
                                     size_t groups, size_t seq, size_t head_dim,
                                     float scale, bool add_q, bool add_k,
                                     bool add_v, bool recompute,
                                     cudaStream_t stream, HeadLayout in_layout,
                                     HeadLayout out_layout,
                                     HeadLayout dout_layout,
                                     HeadLayout grad_layout) {
    in_layout = resolve_layout(in_layout, head_dim);
    out_layout = resolve_layout(out_layout, head_dim);
    dout_layout = resolve_layout(dout_layout, head_dim);
    grad_layout = resolve_layout(grad_layout, head_dim);
    const unsigned threads = unsigned((seq + 31) / 32 * 32);
    const size_t bytes = (4 * seq * head_dim + seq * (seq | 1)) * sizeof(float);
    bool launched = false;
#define CALL(HD)                                                               \
    if (fit_shared(attention_small_backward_kernel<HD>, bytes)) {              \
        attention_small_backward_kernel<HD>                                    \
            <<<unsigned(groups), threads, bytes, stream>>>(                    \
                q, k, v, probabilities, out, dout, dq, dk, dv, int(seq),       \
                scale, add_q, add_k, add_v, recompute, in_layout, out_layout,  \
                dout_layout, grad_layout);                                     \
        launched = true;                                                       \
    }
    VITB200_DISPATCH_HD(head_dim, CALL)
#undef CALL
    g_kernel_launches += launched ? 1 : 0;
    return launched;
}

}  // namespace vitb200
