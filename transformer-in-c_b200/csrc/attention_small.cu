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

// Cooperative copy of a contiguous [rows, HD] block into shared memory.
template <int HD>
__device__ __forceinline__ void load_rows(const float *__restrict__ source,
                                          float *tile, int rows) {
    const int vectors = rows * HD / 4;
    const float4 *from = reinterpret_cast<const float4 *>(source);
    float4 *to = reinterpret_cast<float4 *>(tile);
    for (int i = threadIdx.x; i < vectors; i += blockDim.x) {
        to[i] = __ldcs(from + i);
    }
}

template <int HD>
__global__ void attention_small_forward_kernel(
    const float *__restrict__ q, const float *__restrict__ k,
    const float *__restrict__ v, float *__restrict__ p, float *__restrict__ out,
    int seq, float scale) {
    extern __shared__ __align__(16) float shared[];
    const int pitch = seq | 1;
    float *k_tile = shared;
    float *v_tile = k_tile + seq * HD;
    float *p_tile = v_tile + seq * HD;
    const size_t group = blockIdx.x;
    const size_t base = group * seq * HD;
    load_rows<HD>(k + base, k_tile, seq);
    load_rows<HD>(v + base, v_tile, seq);
    const int row = threadIdx.x;
    float query[HD];
    if (row < seq) {
#pragma unroll
        for (int d = 0; d < HD; d += 4) {
            const float4 x =
                __ldcs(reinterpret_cast<const float4 *>(q + base + row * HD + d));
            query[d] = x.x; query[d + 1] = x.y; query[d + 2] = x.z; query[d + 3] = x.w;
        }
    }
    __syncthreads();
    if (row < seq) {
        float *scores = p_tile + row * pitch;
        float maximum = -FLT_MAX;
        for (int j = 0; j < seq; ++j) {
            const float *key = k_tile + j * HD;
            float dot = 0.0f;
#pragma unroll
            for (int d = 0; d < HD; ++d) {
                dot += query[d] * key[d];
            }
            dot *= scale;
            scores[j] = dot;
            maximum = fmaxf(maximum, dot);
        }
        float denominator = 0.0f;
        for (int j = 0; j < seq; ++j) {
            const float e = expf(scores[j] - maximum);
            scores[j] = e;
            denominator += e;
        }
        float result[HD];
#pragma unroll
        for (int d = 0; d < HD; ++d) {
            result[d] = 0.0f;
        }
        for (int j = 0; j < seq; ++j) {
            const float probability = scores[j] / denominator;
            scores[j] = probability;
            const float *value = v_tile + j * HD;
#pragma unroll
            for (int d = 0; d < HD; ++d) {
                result[d] += probability * value[d];
            }
        }
#pragma unroll
        for (int d = 0; d < HD; d += 4) {
            *reinterpret_cast<float4 *>(out + base + row * HD + d) =
                make_float4(result[d], result[d + 1], result[d + 2], result[d + 3]);
        }
    }
    __syncthreads();
    float *p_group = p + group * seq * seq;
    for (int i = threadIdx.x; i < seq * seq; i += blockDim.x) {
        p_group[i] = p_tile[(i / seq) * pitch + i % seq];
    }
}

template <int HD>
__global__ void attention_small_backward_kernel(
    const float *__restrict__ q, const float *__restrict__ k,
    const float *__restrict__ v, const float *__restrict__ p,
    const float *__restrict__ out, const float *__restrict__ dout,
    float *__restrict__ dq, float *__restrict__ dk, float *__restrict__ dv,
    int seq, float scale, bool add_q, bool add_k, bool add_v) {
    extern __shared__ __align__(16) float shared[];
    const int pitch = seq | 1;
    float *q_tile = shared;
    float *k_tile = q_tile + seq * HD;
    float *v_tile = k_tile + seq * HD;
    float *do_tile = v_tile + seq * HD;
    float *p_tile = do_tile + seq * HD;
    const size_t group = blockIdx.x;
    const size_t base = group * seq * HD;
    load_rows<HD>(q + base, q_tile, seq);
    load_rows<HD>(k + base, k_tile, seq);
    load_rows<HD>(v + base, v_tile, seq);
    load_rows<HD>(dout + base, do_tile, seq);
    const float *p_group = p + group * seq * seq;
    for (int i = threadIdx.x; i < seq * seq; i += blockDim.x) {
        p_tile[(i / seq) * pitch + i % seq] = __ldcs(p_group + i);
    }
    const int row = threadIdx.x;
    float row_dot = 0.0f;
    if (row < seq) {
#pragma unroll
        for (int d = 0; d < HD; d += 4) {
            const float4 o =
                __ldcs(reinterpret_cast<const float4 *>(out + base + row * HD + d));
            const float4 g =
                __ldcs(reinterpret_cast<const float4 *>(dout + base + row * HD + d));
            row_dot += (o.x * g.x + o.y * g.y) + (o.z * g.z + o.w * g.w);
        }
    }
    __syncthreads();
    float acc[HD];
    // Columns: dV_j = sum_i P_ij dO_i.
    if (row < seq) {
#pragma unroll
        for (int d = 0; d < HD; ++d) {
            acc[d] = 0.0f;
        }
        for (int i = 0; i < seq; ++i) {
            const float probability = p_tile[i * pitch + row];
            const float *g = do_tile + i * HD;
#pragma unroll
            for (int d = 0; d < HD; ++d) {
                acc[d] += probability * g[d];
            }
        }
#pragma unroll
        for (int d = 0; d < HD; d += 4) {
            float4 *target = reinterpret_cast<float4 *>(dv + base + row * HD + d);
            float4 t = add_v ? *target : make_float4(0.f, 0.f, 0.f, 0.f);
            t.x += acc[d]; t.y += acc[d + 1]; t.z += acc[d + 2]; t.w += acc[d + 3];
            *target = t;
        }
    }
    __syncthreads();
    // Rows: score gradients in place over P, then dQ_i.
    if (row < seq) {
        float g[HD];
#pragma unroll
        for (int d = 0; d < HD; ++d) {
            g[d] = do_tile[row * HD + d];
            acc[d] = 0.0f;
        }
        float *scores = p_tile + row * pitch;
        for (int j = 0; j < seq; ++j) {
            const float *value = v_tile + j * HD;
            float dp = 0.0f;
#pragma unroll
            for (int d = 0; d < HD; ++d) {
                dp += g[d] * value[d];
            }
            const float ds = scale * scores[j] * (dp - row_dot);
            scores[j] = ds;
            const float *key = k_tile + j * HD;
#pragma unroll
            for (int d = 0; d < HD; ++d) {
                acc[d] += ds * key[d];
            }
        }
#pragma unroll
        for (int d = 0; d < HD; d += 4) {
            float4 *target = reinterpret_cast<float4 *>(dq + base + row * HD + d);
            float4 t = add_q ? *target : make_float4(0.f, 0.f, 0.f, 0.f);
            t.x += acc[d]; t.y += acc[d + 1]; t.z += acc[d + 2]; t.w += acc[d + 3];
            *target = t;
        }
    }
    __syncthreads();
    // Columns: dK_j = sum_i dS_ij Q_i.
    if (row < seq) {
#pragma unroll
        for (int d = 0; d < HD; ++d) {
            acc[d] = 0.0f;
        }
        for (int i = 0; i < seq; ++i) {
            const float ds = p_tile[i * pitch + row];
            const float *query = q_tile + i * HD;
#pragma unroll
            for (int d = 0; d < HD; ++d) {
                acc[d] += ds * query[d];
            }
        }
#pragma unroll
        for (int d = 0; d < HD; d += 4) {
            float4 *target = reinterpret_cast<float4 *>(dk + base + row * HD + d);
            float4 t = add_k ? *target : make_float4(0.f, 0.f, 0.f, 0.f);
            t.x += acc[d]; t.y += acc[d + 1]; t.z += acc[d + 2]; t.w += acc[d + 3];
            *target = t;
        }
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
                                    size_t head_dim, float scale,
                                    cudaStream_t stream) {
    const unsigned threads = unsigned((seq + 31) / 32 * 32);
    const size_t bytes = (2 * seq * head_dim + seq * (seq | 1)) * sizeof(float);
    bool launched = false;
#define CALL(HD)                                                               \
    if (fit_shared(attention_small_forward_kernel<HD>, bytes)) {               \
        attention_small_forward_kernel<HD>                                     \
            <<<unsigned(groups), threads, bytes, stream>>>(                    \
                q, k, v, probabilities, out, int(seq), scale);                 \
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
                                     bool add_v, cudaStream_t stream) {
    const unsigned threads = unsigned((seq + 31) / 32 * 32);
    const size_t bytes = (4 * seq * head_dim + seq * (seq | 1)) * sizeof(float);
    bool launched = false;
#define CALL(HD)                                                               \
    if (fit_shared(attention_small_backward_kernel<HD>, bytes)) {              \
        attention_small_backward_kernel<HD>                                    \
            <<<unsigned(groups), threads, bytes, stream>>>(                    \
                q, k, v, probabilities, out, dout, dq, dk, dv, int(seq),       \
                scale, add_q, add_k, add_v);                                                      \
        launched = true;                                                       \
    }
    VITB200_DISPATCH_HD(head_dim, CALL)
#undef CALL
    g_kernel_launches += launched ? 1 : 0;
    return launched;
}

}  // namespace vitb200
