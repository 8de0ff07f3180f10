// Bidirectional multi-head attention on head-major tensors, with the full
// probability matrix materialised (the host keeps it as a tensor and hands it
// back to the backward pass; reference src/ops.c:1297-1355, :1381-1441).
//
// Work decomposition: one block per (group, tile of 32 rows), 256 threads;
// thread t serves row t/8 of the tile and, inside any 32-wide tile of the
// other axis, the four entries (t%8) + 8j.  Operand tiles are staged in
// shared memory with an odd row pitch, so the eight threads of a row read
// eight different banks and the four rows of a warp broadcast.
//
//   forward   scores -> row max -> denominators -> P, O = P V      (3 sweeps)
//   backward  D_i = dO_i . O_i
//             query-major kernel: dP = dO V^T, dS = scale P (dP - D), dQ += dS K
//             key-major kernel:   same dS recomputed,  dK += dS^T Q, dV += P^T dO
#include "kernels.h"
#include "gemm.h"
#include "../../include/vitb200.h"
#include "device_util.cuh"

#include <cfloat>

namespace vitb200 {
namespace {

constexpr int kTile = 32;          // rows per block, and keys per sweep step
constexpr int kLanesPerRow = 8;    // threads cooperating on one row
constexpr int kThreads = kTile * kLanesPerRow;

__device__ __forceinline__ float lanes8_sum(float v) {
    v += __shfl_xor_sync(kFullMask, v, 1);
    v += __shfl_xor_sync(kFullMask, v, 2);
    v += __shfl_xor_sync(kFullMask, v, 4);
    return v;
}

__device__ __forceinline__ float lanes8_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(kFullMask, v, 1));
    v = fmaxf(v, __shfl_xor_sync(kFullMask, v, 2));
    v = fmaxf(v, __shfl_xor_sync(kFullMask, v, 4));
    return v;
}

// Copies rows [row0, row0+32) x head_dim of a [seq, head_dim] matrix into a
// shared tile with pitch head_dim+1; rows past `seq` become zeros.
__device__ __forceinline__ void stage_tile(const float *__restrict__ base,
                                           float *tile, int row0, int seq,
                                           int head_dim) {
    const int pitch = head_dim + 1;
    for (int i = threadIdx.x; i < kTile * head_dim; i += kThreads) {
        const int r = i / head_dim;
        const int d = i % head_dim;
        tile[r * pitch + d] =
            row0 + r < seq ? base[size_t(row0 + r) * head_dim + d] : 0.0f;
    }
}

__device__ __forceinline__ float dot_rows(const float *a, const float *b,
                                          int head_dim) {
    float sum = 0.0f;
    for (int d = 0; d < head_dim; ++d) {
        sum += a[d] * b[d];
    }
    return sum;
}

template <int NI>
__global__ void __launch_bounds__(kThreads)
attention_forward_kernel(const float *__restrict__ q,
                         const float *__restrict__ k,
                         const float *__restrict__ v, float *__restrict__ p,
                         float *__restrict__ out, int seq, int head_dim,
                         float scale) {
    extern __shared__ float shared[];
    const int pitch = head_dim + 1;
    float *q_tile = shared;
    float *kv_tile = q_tile + kTile * pitch;
    float *p_tile = kv_tile + kTile * pitch;  // [32][33]

    const size_t group = blockIdx.x;
    const int row0 = blockIdx.y * kTile;
    const int r = threadIdx.x / kLanesPerRow;
    const int sub = threadIdx.x % kLanesPerRow;
    const int row = row0 + r;
    const bool live = row < seq;
    const float *gq = q + group * seq * head_dim;
    const float *gk = k + group * seq * head_dim;
    const float *gv = v + group * seq * head_dim;
    float *prow = p + (group * seq + (live ? row : 0)) * seq;

    stage_tile(gq, q_tile, row0, seq, head_dim);

    // Sweep 1: raw scaled scores to global memory, running row maximum.
    float maximum = -FLT_MAX;
    for (int key0 = 0; key0 < seq; key0 += kTile) {
        __syncthreads();
        stage_tile(gk, kv_tile, key0, seq, head_dim);
        __syncthreads();
#pragma unroll
        for (int j = 0; j < kTile / kLanesPerRow; ++j) {
            const int kk = sub + kLanesPerRow * j;
            if (live && key0 + kk < seq) {
                const float score =
                    scale * dot_rows(q_tile + r * pitch, kv_tile + kk * pitch,
                                     head_dim);
                prow[key0 + kk] = score;
                maximum = fmaxf(maximum, score);
            }
        }
    }
    maximum = lanes8_max(maximum);

    // Sweep 2: denominators (each thread re-reads only what it wrote).
    float denominator = 0.0f;
    if (live) {
        for (int key = sub; key < seq; key += kLanesPerRow) {
            denominator += expf(prow[key] - maximum);
        }
    }
    denominator = lanes8_sum(denominator);

    // Sweep 3: probabilities and O = P V.
    float acc[NI];
#pragma unroll
    for (int i = 0; i < NI; ++i) {
        acc[i] = 0.0f;
    }
    for (int key0 = 0; key0 < seq; key0 += kTile) {
        __syncthreads();
        stage_tile(gv, kv_tile, key0, seq, head_dim);
#pragma unroll
        for (int j = 0; j < kTile / kLanesPerRow; ++j) {
            const int kk = sub + kLanesPerRow * j;
            float probability = 0.0f;
            if (live && key0 + kk < seq) {
                probability = expf(prow[key0 + kk] - maximum) / denominator;
                prow[key0 + kk] = probability;
            }
            p_tile[r * (kTile + 1) + kk] = probability;
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            const int d = sub + kLanesPerRow * i;
            if (d < head_dim) {
                float sum = acc[i];
                for (int kk = 0; kk < kTile; ++kk) {
                    sum += p_tile[r * (kTile + 1) + kk] * kv_tile[kk * pitch + d];
                }
                acc[i] = sum;
            }
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            const int d = sub + kLanesPerRow * i;
            if (d < head_dim) {
                out[(group * seq + row) * head_dim + d] = acc[i];
            }
        }
    }
}

// D_i = dO_i . O_i for every attention row; one warp per row.
__global__ void row_dots_kernel(const float *__restrict__ a,
                                const float *__restrict__ b,
                                float *__restrict__ out, size_t rows,
                                int head_dim) {
    const int lane = threadIdx.x & 31;
    const size_t warp = (size_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const size_t warps = (size_t(gridDim.x) * blockDim.x) >> 5;
    for (size_t row = warp; row < rows; row += warps) {
        float sum = 0.0f;
        for (int d = lane; d < head_dim; d += 32) {
            sum += a[row * head_dim + d] * b[row * head_dim + d];
        }
        sum = warp_sum(sum);
        if (lane == 0) {
            out[row] = sum;
        }
    }
}

template <int NI>
__global__ void __launch_bounds__(kThreads)
attention_backward_query_kernel(const float *__restrict__ k,
                                const float *__restrict__ v,
                                const float *__restrict__ p,
                                const float *__restrict__ dout,
                                const float *__restrict__ row_dots,
                                float *__restrict__ dq, int seq, int head_dim,
                                float scale, bool add_q) {
    extern __shared__ float shared[];
    const int pitch = head_dim + 1;
    float *do_tile = shared;
    float *k_tile = do_tile + kTile * pitch;
    float *v_tile = k_tile + kTile * pitch;
    float *s_tile = v_tile + kTile * pitch;  // [32][33]

    const size_t group = blockIdx.x;
    const int row0 = blockIdx.y * kTile;
    const int r = threadIdx.x / kLanesPerRow;
    const int sub = threadIdx.x % kLanesPerRow;
    const int row = row0 + r;
    const bool live = row < seq;
    const size_t base = group * seq * head_dim;
    const float *prow = p + (group * seq + (live ? row : 0)) * seq;
    const float dot = live ? row_dots[group * seq + row] : 0.0f;

    stage_tile(dout + base, do_tile, row0, seq, head_dim);
    float acc[NI];
#pragma unroll
    for (int i = 0; i < NI; ++i) {
        acc[i] = 0.0f;
    }
    for (int key0 = 0; key0 < seq; key0 += kTile) {
        __syncthreads();
        stage_tile(k + base, k_tile, key0, seq, head_dim);
        stage_tile(v + base, v_tile, key0, seq, head_dim);
        __syncthreads();
#pragma unroll
        for (int j = 0; j < kTile / kLanesPerRow; ++j) {
            const int kk = sub + kLanesPerRow * j;
            float score_grad = 0.0f;
            if (live && key0 + kk < seq) {
                const float dp = dot_rows(do_tile + r * pitch,
                                          v_tile + kk * pitch, head_dim);
                score_grad = scale * prow[key0 + kk] * (dp - dot);
            }
            s_tile[r * (kTile + 1) + kk] = score_grad;
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            const int d = sub + kLanesPerRow * i;
            if (d < head_dim) {
                float sum = acc[i];
                for (int kk = 0; kk < kTile; ++kk) {
                    sum += s_tile[r * (kTile + 1) + kk] * k_tile[kk * pitch + d];
                }
                acc[i] = sum;
            }
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            const int d = sub + kLanesPerRow * i;
            if (d < head_dim) {
                float *target = dq + base + size_t(row) * head_dim + d;
                *target = (add_q ? *target : 0.0f) + acc[i];
            }
        }
    }
}

template <int NI>
__global__ void __launch_bounds__(kThreads)
attention_backward_key_kernel(const float *__restrict__ q,
                              const float *__restrict__ v,
                              const float *__restrict__ p,
                              const float *__restrict__ dout,
                              const float *__restrict__ row_dots,
                              float *__restrict__ dk, float *__restrict__ dv,
                              int seq, int head_dim, float scale, bool add_k,
                              bool add_v) {
    extern __shared__ float shared[];
    const int pitch = head_dim + 1;
    float *v_tile = shared;                     // this block's keys
    float *q_tile = v_tile + kTile * pitch;     // current query tile
    float *do_tile = q_tile + kTile * pitch;
    float *p_tile = do_tile + kTile * pitch;    // [query][key], pitch 33
    float *s_tile = p_tile + kTile * (kTile + 1);
    float *dots = s_tile + kTile * (kTile + 1); // [32]

    const size_t group = blockIdx.x;
    const int key0 = blockIdx.y * kTile;
    const int r = threadIdx.x / kLanesPerRow;   // key within the tile
    const int sub = threadIdx.x % kLanesPerRow;
    const int key = key0 + r;
    const bool live = key < seq;
    const size_t base = group * seq * head_dim;
    const float *gp = p + group * seq * seq;

    stage_tile(v + base, v_tile, key0, seq, head_dim);
    float acc_k[NI], acc_v[NI];
#pragma unroll
    for (int i = 0; i < NI; ++i) {
        acc_k[i] = 0.0f;
        acc_v[i] = 0.0f;
    }
    for (int query0 = 0; query0 < seq; query0 += kTile) {
        __syncthreads();
        stage_tile(q + base, q_tile, query0, seq, head_dim);
        stage_tile(dout + base, do_tile, query0, seq, head_dim);
        // Probability tile, read along rows of P so the loads coalesce.
        for (int i = threadIdx.x; i < kTile * kTile; i += kThreads) {
            const int qi = i / kTile;
            const int kj = i % kTile;
            p_tile[qi * (kTile + 1) + kj] =
                (query0 + qi < seq && key0 + kj < seq)
                    ? gp[size_t(query0 + qi) * seq + key0 + kj]
                    : 0.0f;
        }
        if (threadIdx.x < kTile) {
            dots[threadIdx.x] = query0 + threadIdx.x < seq
                ? row_dots[group * seq + query0 + threadIdx.x]
                : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < kTile / kLanesPerRow; ++j) {
            const int qi = sub + kLanesPerRow * j;
            const float probability = p_tile[qi * (kTile + 1) + r];
            const float dp = dot_rows(do_tile + qi * pitch, v_tile + r * pitch,
                                      head_dim);
            s_tile[qi * (kTile + 1) + r] =
                scale * probability * (dp - dots[qi]);
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            const int d = sub + kLanesPerRow * i;
            if (d < head_dim) {
                float sum_k = acc_k[i], sum_v = acc_v[i];
                for (int qi = 0; qi < kTile; ++qi) {
                    sum_k += s_tile[qi * (kTile + 1) + r] * q_tile[qi * pitch + d];
                    sum_v += p_tile[qi * (kTile + 1) + r] * do_tile[qi * pitch + d];
                }
                acc_k[i] = sum_k;
                acc_v[i] = sum_v;
            }
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            const int d = sub + kLanesPerRow * i;
            if (d < head_dim) {
                float *target_k = dk + base + size_t(key) * head_dim + d;
                float *target_v = dv + base + size_t(key) * head_dim + d;
                *target_k = (add_k ? *target_k : 0.0f) + acc_k[i];
                *target_v = (add_v ? *target_v : 0.0f) + acc_v[i];
            }
        }
    }
}

template <typename Kernel>
void allow_shared(Kernel kernel, size_t bytes) {
    if (bytes > 48 * 1024) {
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(bytes));
    }
}

#define VITB200_DISPATCH_NI(head_dim, CALL)                                    \
    do {                                                                       \
        const int slots = (int(head_dim) + kLanesPerRow - 1) / kLanesPerRow;   \
        if (slots <= 1) { CALL(1); }                                           \
        else if (slots <= 2) { CALL(2); }                                      \
        else if (slots <= 4) { CALL(4); }                                      \
        else if (slots <= 8) { CALL(8); }                                      \
        else { CALL(16); }                                                     \
    } while (0)

}  // namespace

void launch_attention_forward(const float *q, const float *k, const float *v,
                              float *probabilities, float *out, size_t groups,
                              size_t seq, size_t head_dim, float scale,
                              int precision, cudaStream_t stream) {
    // Short sequences are limited by shared-memory and instruction traffic,
    // not by arithmetic: the FP32 whole-group kernel is as fast there and
    // exact, so tensor cores are used for them only on explicit request.
    const double work = double(groups) * seq * seq * head_dim;
    const bool short_sequence = attention_small_supported(seq, head_dim);
    if (attention_mma_supported(head_dim) &&
        (precision == VITB200_PRECISION_TF32 ||
         (!short_sequence && prefer_tensor_cores(precision, work))) &&
        launch_attention_mma_forward(q, k, v, probabilities, out, groups, seq,
                                     head_dim, scale, stream)) {
        return;
    }
    if (attention_small_supported(seq, head_dim) &&
        launch_attention_small_forward(q, k, v, probabilities, out, groups, seq,
                                       head_dim, scale, true, true, stream)) {
        return;
    }
    const dim3 grid(static_cast<unsigned>(groups),
                    static_cast<unsigned>((seq + kTile - 1) / kTile));
    const size_t pitch = head_dim + 1;
    const size_t bytes = (2 * kTile * pitch + kTile * (kTile + 1)) * sizeof(float);
#define CALL(NI)                                                               \
    allow_shared(attention_forward_kernel<NI>, bytes);                         \
    attention_forward_kernel<NI><<<grid, kThreads, bytes, stream>>>(           \
        q, k, v, probabilities, out, int(seq), int(head_dim), scale)
    VITB200_DISPATCH_NI(head_dim, CALL);
#undef CALL
    ++g_kernel_launches;
}

void launch_attention_backward(const float *q, const float *k, const float *v,
                               const float *probabilities, const float *out,
                               const float *dout, float *dq, float *dk,
                               float *dv, float *row_dots, size_t groups,
                               size_t seq, size_t head_dim, float scale,
                               bool add_q, bool add_k, bool add_v,
                               int precision, cudaStream_t stream) {
    const double work = double(groups) * seq * seq * head_dim;
    const bool short_sequence = attention_small_supported(seq, head_dim);
    if (attention_mma_supported(head_dim) &&
        (precision == VITB200_PRECISION_TF32 ||
         (!short_sequence && prefer_tensor_cores(precision, work))) &&
        launch_attention_mma_backward(q, k, v, probabilities, nullptr, out,
                                      dout, dq, dk, dv, row_dots, groups, seq,
                                      head_dim,
                                      scale, add_q, add_k, add_v, stream)) {
        return;
    }
    if (attention_small_supported(seq, head_dim) &&
        launch_attention_small_backward(q, k, v, probabilities, out, dout, dq,
                                        dk, dv, groups, seq, head_dim, scale,
                                        add_q, add_k, add_v, false, stream)) {
        return;
    }
    const size_t rows = groups * seq;
    row_dots_kernel<<<stream_grid(rows * 32), kStreamThreads, 0, stream>>>(
        dout, out, row_dots, rows, int(head_dim));
    const dim3 grid(static_cast<unsigned>(groups),
                    static_cast<unsigned>((seq + kTile - 1) / kTile));
    const size_t pitch = head_dim + 1;
    const size_t query_bytes =
        (3 * kTile * pitch + kTile * (kTile + 1)) * sizeof(float);
    const size_t key_bytes =
        (3 * kTile * pitch + 2 * kTile * (kTile + 1) + kTile) * sizeof(float);
#define CALL(NI)                                                               \
    allow_shared(attention_backward_query_kernel<NI>, query_bytes);            \
    attention_backward_query_kernel<NI><<<grid, kThreads, query_bytes, stream>>>(\
        k, v, probabilities, dout, row_dots, dq, int(seq), int(head_dim),      \
        scale, add_q);                                                              \
    allow_shared(attention_backward_key_kernel<NI>, key_bytes);                \
    attention_backward_key_kernel<NI><<<grid, kThreads, key_bytes, stream>>>(  \
        q, v, probabilities, dout, row_dots, dk, dv, int(seq), int(head_dim),  \
        scale, add_k, add_v)
    VITB200_DISPATCH_NI(head_dim, CALL);
#undef CALL
    g_kernel_launches += 3;
}

}  // namespace vitb200
